// The sm_100a Atom: the two datapath primitives every collective is built from.
//
//   Atom::copy(dst, src, bytes)     one CTA moves an aligned slice; either side may be
//                                   peer memory reached over NVLink
//   Atom::reduce<T, Op>(args)       one CTA combines the same slice of every rank's
//                                   staging buffer in ascending rank order with fp32
//                                   accumulation, or lets the NVSwitch do it with
//                                   multimem.ld_reduce, and writes the result to local
//                                   memory and/or broadcasts it with multimem.st
//
// Parity: the Atom contract of csrc/include/purlin/atom.cuh:9-12 and the sm_100
// datapath of cortex.cuh:9-59 / ligament.cuh:20-152 in the reference. This is a
// Blackwell-only implementation: copies move 32 bytes per access (ld/st.global.v8).
// Reductions load 16 bytes per peer per access: a 32-byte form was built and measured
// on B200 over NVLink (2 GPUs, reduce-scatter of 32 MiB / 256 MiB: 83 / 507 us against
// 64 / 331 us) and, compiled into the same kernel, pushed every reduce instantiation
// into register spills, so it was taken out again; multimem.ld_reduce is 128 bits wide
// at most in any case. Arithmetic is packed f32x2; the number of accesses in flight per
// thread is a knob chosen by the tuning policy.
#pragma once
#include "math.cuh"
#include "signal.cuh"

namespace purlin {

struct alignas(32) Vec32 { uint32_t x[8]; };
struct alignas(16) Vec16 { uint32_t x[4]; };

PURLIN_D Vec32 ld32(const void* p) {
  Vec32 v;
  asm volatile("ld.global.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]), "=r"(v.x[4]), "=r"(v.x[5]), "=r"(v.x[6]), "=r"(v.x[7])
               : "l"(p) : "memory");
  return v;
}
PURLIN_D void st32(void* p, const Vec32& v) {
  asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.x[0]), "r"(v.x[1]), "r"(v.x[2]),
               "r"(v.x[3]), "r"(v.x[4]), "r"(v.x[5]), "r"(v.x[6]), "r"(v.x[7]) : "memory");
}
PURLIN_D Vec16 ld16(const void* p) {
  Vec16 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]) : "l"(p) : "memory");
  return v;
}
PURLIN_D void st16(void* p, const Vec16& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x[0]), "r"(v.x[1]), "r"(v.x[2]), "r"(v.x[3]) : "memory");
}

// ---- NVLS: reduction and broadcast performed by the NVSwitch on a multicast address ----
template <DType T, ReduceOp Op> struct MultimemReducible { static constexpr bool value = false; };
template <> struct MultimemReducible<DType::bf16, ReduceOp::add> { static constexpr bool value = true; };
template <> struct MultimemReducible<DType::fp16, ReduceOp::add> { static constexpr bool value = true; };
template <> struct MultimemReducible<DType::fp32, ReduceOp::add> { static constexpr bool value = true; };
template <> struct MultimemReducible<DType::bf16, ReduceOp::max> { static constexpr bool value = true; };
template <> struct MultimemReducible<DType::fp16, ReduceOp::max> { static constexpr bool value = true; };

template <DType T, ReduceOp Op> PURLIN_D Vec16 multimemLdReduce(const void* mc) {
  Vec16 v;
  if constexpr (T == DType::bf16 && Op == ReduceOp::add)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]) : "l"(mc) : "memory");
  else if constexpr (T == DType::fp16 && Op == ReduceOp::add)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]) : "l"(mc) : "memory");
  else if constexpr (T == DType::fp32 && Op == ReduceOp::add)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]) : "l"(mc) : "memory");
  else if constexpr (T == DType::bf16 && Op == ReduceOp::max)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]) : "l"(mc) : "memory");
  else if constexpr (T == DType::fp16 && Op == ReduceOp::max)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.f16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]) : "l"(mc) : "memory");
  else
    v = Vec16{};
  return v;
}
PURLIN_D void multimemSt(void* mc, const Vec16& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x[0]), "r"(v.x[1]), "r"(v.x[2]), "r"(v.x[3]) : "memory");
}

struct ReduceArgs {
  const unsigned char* const* srcs = nullptr;  // one pointer per rank, ascending rank order (unicast path)
  const unsigned char* mcSrc = nullptr;        // multicast alias of the same slice (NVLS path), or null
  unsigned char* dst = nullptr;                // local result, or null
  unsigned char* seam = nullptr;               // second local result (composition seam), or null
  unsigned char* mcSeam = nullptr;             // multicast result: the NVSwitch stores it on every rank, or null
  size_t bytes = 0;
  int world = 0;
};

template <int Threads = 256, int Unroll = 4, int MmDepth = 4>
struct AtomSm100 {
  static constexpr int THREADS = Threads;
  static constexpr int UNROLL = Unroll;
  static constexpr int MM_DEPTH = MmDepth;
  static constexpr int GMEM_ACCESS_ALIGNMENT_BYTES = int(kAccessAlign);

  // One CTA copies `bytes` (a multiple of 16; 32 gives the widest accesses). `unroll` = 32-byte accesses in
  // flight per thread (4 or 8): bytes in flight per CTA = threads x unroll x 32.
  static PURLIN_D void copy(unsigned char* dst, const unsigned char* src, size_t bytes, int unroll = Unroll) {
    if (unroll >= 8) copyImpl<8>(dst, src, bytes);
    else copyImpl<4>(dst, src, bytes);
  }

  template <int U>
  static PURLIN_D void copyImpl(unsigned char* dst, const unsigned char* src, size_t bytes) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const bool wide = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 31u) == 0;
    size_t done = 0;
    if (wide) {
      const size_t n = bytes / 32;
      size_t i = tid;
      for (; i + size_t(U - 1) * nt < n; i += size_t(U) * nt) {
        Vec32 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = ld32(src + (i + size_t(u) * nt) * 32);
#pragma unroll
        for (int u = 0; u < U; ++u) st32(dst + (i + size_t(u) * nt) * 32, v[u]);
      }
      for (; i < n; i += nt) st32(dst + i * 32, ld32(src + i * 32));
      done = n * 32;
    } else if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0) {
      const size_t n = bytes / 16;
      for (size_t i = tid; i < n; i += nt) st16(dst + i * 16, ld16(src + i * 16));
      done = n * 16;
    }
    for (size_t i = done + tid; i < bytes; i += nt) dst[i] = src[i];
  }

  // One CTA reduces `bytes` (a multiple of 16) of every rank's slice. `mmDepth` = multimem loads in flight per
  // thread on the NVLS path (1, 2, 4 or 8).
  template <DType T, ReduceOp Op>
  static PURLIN_D void reduce(const ReduceArgs& a, int mmDepth = MmDepth) {
    if constexpr (MultimemReducible<T, Op>::value) {
      if (a.mcSrc != nullptr) {
        if (mmDepth >= 8) reduceMultimem<T, Op, 8>(a);
        else if (mmDepth >= 4) reduceMultimem<T, Op, 4>(a);
        else if (mmDepth >= 2) reduceMultimem<T, Op, 2>(a);
        else reduceMultimem<T, Op, 1>(a);
        return;
      }
    }
    // eight 16-byte loads in flight per thread: peers-per-batch x vectors-per-iteration = 8
    if (a.world <= 2) reduceUnicast<T, Op, 2>(a);
    else if (a.world <= 4) reduceUnicast<T, Op, 4>(a);
    else reduceUnicast<T, Op, 8>(a);
  }

  template <DType T, ReduceOp Op, int D>
  static PURLIN_D void reduceMultimem(const ReduceArgs& a) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const size_t n = a.bytes / 16;
    size_t i = tid;
    for (; i + size_t(D - 1) * nt < n; i += size_t(D) * nt) {
      Vec16 v[D];
#pragma unroll
      for (int d = 0; d < D; ++d) v[d] = multimemLdReduce<T, Op>(a.mcSrc + (i + size_t(d) * nt) * 16);
#pragma unroll
      for (int d = 0; d < D; ++d) emit(a, (i + size_t(d) * nt) * 16, v[d]);
    }
    for (; i < n; i += nt) emit(a, i * 16, multimemLdReduce<T, Op>(a.mcSrc + i * 16));
  }

  // Worlds of at most 8 ranks: every peer's copy of U = 8 / WB consecutive vectors is requested before any is
  // consumed (8 loads of 16 bytes in flight per thread); accumulation stays in ascending rank order.
  // Larger worlds take peers in batches of 8 with one vector per iteration.
  template <DType T, ReduceOp Op, int WB>
  static PURLIN_D void reduceUnicast(const ReduceArgs& a) {
    constexpr int U = 8 / WB;
    const int tid = threadIdx.x, nt = blockDim.x;
    const size_t n = a.bytes / 16;
    if (a.world <= WB) {
      for (size_t i0 = tid; i0 < n; i0 += size_t(U) * nt) {
        Vec16 v[U][WB];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int b = 0; b < WB; ++b)
            if (b < a.world && i0 + size_t(u) * nt < n) v[u][b] = ld16(a.srcs[b] + (i0 + size_t(u) * nt) * 16);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + size_t(u) * nt >= n) break;
          Acc<T> lo, hi;
#pragma unroll
          for (int e = 0; e < ElemTraits<T>::perWord; ++e) lo.v[e] = hi.v[e] = identity<Op>();
#pragma unroll
          for (int b = 0; b < WB; ++b)
            if (b < a.world) {
              accumulate<T, Op>(lo, unpack<T>(uint64_t(v[u][b].x[0]) | (uint64_t(v[u][b].x[1]) << 32)));
              accumulate<T, Op>(hi, unpack<T>(uint64_t(v[u][b].x[2]) | (uint64_t(v[u][b].x[3]) << 32)));
            }
          const uint64_t w0 = pack<T>(lo), w1 = pack<T>(hi);
          emit(a, (i0 + size_t(u) * nt) * 16, Vec16{{uint32_t(w0), uint32_t(w0 >> 32), uint32_t(w1), uint32_t(w1 >> 32)}});
        }
      }
      return;
    }
    for (size_t i = tid; i < n; i += nt) {
      Acc<T> lo, hi;
#pragma unroll
      for (int e = 0; e < ElemTraits<T>::perWord; ++e) lo.v[e] = hi.v[e] = identity<Op>();
      for (int q0 = 0; q0 < a.world; q0 += 8) {
        Vec16 v[8];
#pragma unroll
        for (int b = 0; b < 8; ++b)
          if (q0 + b < a.world) v[b] = ld16(a.srcs[q0 + b] + i * 16);
#pragma unroll
        for (int b = 0; b < 8; ++b)
          if (q0 + b < a.world) {
            accumulate<T, Op>(lo, unpack<T>(uint64_t(v[b].x[0]) | (uint64_t(v[b].x[1]) << 32)));
            accumulate<T, Op>(hi, unpack<T>(uint64_t(v[b].x[2]) | (uint64_t(v[b].x[3]) << 32)));
          }
      }
      const uint64_t w0 = pack<T>(lo), w1 = pack<T>(hi);
      emit(a, i * 16, Vec16{{uint32_t(w0), uint32_t(w0 >> 32), uint32_t(w1), uint32_t(w1 >> 32)}});
    }
  }

 private:
  static PURLIN_D void emit(const ReduceArgs& a, size_t off, const Vec16& v) {
    if (a.dst) st16(a.dst + off, v);
    if (a.seam) st16(a.seam + off, v);
    if (a.mcSeam) multimemSt(a.mcSeam + off, v);
  }
};

// Grid-level copy: a set of CTAs splits one region and each copies its share
// (the behaviour of superCopy, csrc/include/purlin/transfer.cuh:9-46).
template <class Atom>
PURLIN_D void superCopy(unsigned char* dst, const unsigned char* src, size_t bytes, int part, int parts, int unroll = 4) {
  const size_t units = bytes / kAccessAlign, tail = bytes - units * kAccessAlign;
  const size_t base = units / size_t(parts), rem = units % size_t(parts), p = size_t(part);
  const size_t begin = (p * base + (p < rem ? p : rem)) * kAccessAlign;
  size_t len = (base + (p < rem ? 1 : 0)) * kAccessAlign;
  if (part == parts - 1) len += tail;
  if (len) Atom::copy(dst + begin, src + begin, len, unroll);
}

}  // namespace purlin
