// Element types, fp32 accumulation and the three reduce operators.
//
// Parity: csrc/include/purlin/math.cuh:11-347 of the reference (add / mul /
// max over bf16, fp16, fp32, fp8 e4m3 and e5m2 with fp32 accumulation) and
// csrc/include/purlin/cortex.cuh:9-23 (packed two-lane fp32 add and multiply,
// which sm_100a executes as one instruction). Written here around one idea: a
// 16-byte vector of any element type unpacks to N floats, is combined in fp32,
// and packs back; the operator is a template tag.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "plan.hpp"

namespace purlin {

template <DType T> struct ElemTraits;
template <> struct ElemTraits<DType::fp32> { static constexpr int perWord = 2; };   // elements per 8-byte word
template <> struct ElemTraits<DType::bf16> { static constexpr int perWord = 4; };
template <> struct ElemTraits<DType::fp16> { static constexpr int perWord = 4; };
template <> struct ElemTraits<DType::fp8e4m3> { static constexpr int perWord = 8; };
template <> struct ElemTraits<DType::fp8e5m2> { static constexpr int perWord = 8; };

// An 8-byte word as floats.
template <DType T> struct Acc { float v[ElemTraits<T>::perWord]; };

template <DType T> PURLIN_D Acc<T> unpack(uint64_t w);
template <DType T> PURLIN_D uint64_t pack(const Acc<T>& a);

template <> PURLIN_D Acc<DType::fp32> unpack<DType::fp32>(uint64_t w) {
  Acc<DType::fp32> a;
  a.v[0] = __uint_as_float(uint32_t(w));
  a.v[1] = __uint_as_float(uint32_t(w >> 32));
  return a;
}
template <> PURLIN_D uint64_t pack<DType::fp32>(const Acc<DType::fp32>& a) {
  return uint64_t(__float_as_uint(a.v[0])) | (uint64_t(__float_as_uint(a.v[1])) << 32);
}
template <> PURLIN_D Acc<DType::bf16> unpack<DType::bf16>(uint64_t w) {
  // bf16 -> fp32 is a 16-bit shift
  Acc<DType::bf16> a;
  const uint32_t lo = uint32_t(w), hi = uint32_t(w >> 32);
  a.v[0] = __uint_as_float(lo << 16);
  a.v[1] = __uint_as_float(lo & 0xffff0000u);
  a.v[2] = __uint_as_float(hi << 16);
  a.v[3] = __uint_as_float(hi & 0xffff0000u);
  return a;
}
template <> PURLIN_D uint64_t pack<DType::bf16>(const Acc<DType::bf16>& a) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a.v[0], a.v[1]);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(a.v[2], a.v[3]);
  return uint64_t(*reinterpret_cast<const uint32_t*>(&lo)) | (uint64_t(*reinterpret_cast<const uint32_t*>(&hi)) << 32);
}
template <> PURLIN_D Acc<DType::fp16> unpack<DType::fp16>(uint64_t w) {
  Acc<DType::fp16> a;
  const uint32_t lo = uint32_t(w), hi = uint32_t(w >> 32);
  const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&lo));
  const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  a.v[0] = f0.x; a.v[1] = f0.y; a.v[2] = f1.x; a.v[3] = f1.y;
  return a;
}
template <> PURLIN_D uint64_t pack<DType::fp16>(const Acc<DType::fp16>& a) {
  const __half2 lo = __floats2half2_rn(a.v[0], a.v[1]);
  const __half2 hi = __floats2half2_rn(a.v[2], a.v[3]);
  return uint64_t(*reinterpret_cast<const uint32_t*>(&lo)) | (uint64_t(*reinterpret_cast<const uint32_t*>(&hi)) << 32);
}
template <__nv_fp8_interpretation_t K, DType T> PURLIN_D Acc<T> unpackFp8(uint64_t w) {
  Acc<T> a;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(__nv_fp8x2_storage_t(w >> (16 * i)), K);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    a.v[2 * i] = f.x;
    a.v[2 * i + 1] = f.y;
  }
  return a;
}
template <__nv_fp8_interpretation_t K, DType T> PURLIN_D uint64_t packFp8(const Acc<T>& a) {
  uint64_t w = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_fp8x2_storage_t s = __nv_cvt_float2_to_fp8x2(make_float2(a.v[2 * i], a.v[2 * i + 1]), __NV_SATFINITE, K);
    w |= uint64_t(s) << (16 * i);
  }
  return w;
}
template <> PURLIN_D Acc<DType::fp8e4m3> unpack<DType::fp8e4m3>(uint64_t w) { return unpackFp8<__NV_E4M3, DType::fp8e4m3>(w); }
template <> PURLIN_D uint64_t pack<DType::fp8e4m3>(const Acc<DType::fp8e4m3>& a) { return packFp8<__NV_E4M3, DType::fp8e4m3>(a); }
template <> PURLIN_D Acc<DType::fp8e5m2> unpack<DType::fp8e5m2>(uint64_t w) { return unpackFp8<__NV_E5M2, DType::fp8e5m2>(w); }
template <> PURLIN_D uint64_t pack<DType::fp8e5m2>(const Acc<DType::fp8e5m2>& a) { return packFp8<__NV_E5M2, DType::fp8e5m2>(a); }

// acc = acc (op) x, two lanes at a time so add and mul become one f32x2 instruction.
template <ReduceOp Op> PURLIN_D float2 combine2(float2 a, float2 b) {
  if constexpr (Op == ReduceOp::add) return __fadd2_rn(a, b);
  else if constexpr (Op == ReduceOp::mul) return __fmul2_rn(a, b);
  else return make_float2(fmaxf(a.x, b.x), fmaxf(a.y, b.y));
}
template <ReduceOp Op> PURLIN_D float identity() {
  if constexpr (Op == ReduceOp::add) return 0.f;
  else if constexpr (Op == ReduceOp::mul) return 1.f;
  else return -INFINITY;
}
template <DType T, ReduceOp Op> PURLIN_D void accumulate(Acc<T>& acc, const Acc<T>& x) {
#pragma unroll
  for (int i = 0; i < ElemTraits<T>::perWord; i += 2) {
    const float2 r = combine2<Op>(make_float2(acc.v[i], acc.v[i + 1]), make_float2(x.v[i], x.v[i + 1]));
    acc.v[i] = r.x;
    acc.v[i + 1] = r.y;
  }
}

}  // namespace purlin
