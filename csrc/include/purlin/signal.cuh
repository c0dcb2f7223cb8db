// Flags, last-arrival counters and bounded waits over peer memory.
//
// Parity: csrc/include/purlin/epoch.cuh:54-130 of the reference (relaxed spin
// followed by an acquire load, release store of a monotonic flag into peer
// memory, self-resetting arrival counter). The difference that matters: the
// reference spins forever, so a missing peer hangs the GPU. Every wait here
// carries a time limit; when it runs out the waiter records where it gave up
// in the context's status word and the whole call unwinds.
#pragma once
#include <cuda_runtime.h>

#include "context.hpp"

namespace purlin {
namespace sig {

PURLIN_D uint64_t ldRelaxedSys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
PURLIN_D uint64_t ldAcquireSys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
PURLIN_D void stReleaseSys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
PURLIN_D void stRelaxedSys(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
PURLIN_D uint32_t ldRelaxedGpu32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
PURLIN_D uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Record the first failure of a call; later failures keep the first record.
PURLIN_D void fail(const Context& ctx, uint32_t code, uint32_t step, uint32_t peer, uint32_t chunk) {
  if (atomicCAS(ctx.status, 0u, code) == 0u) {
    ctx.status[1] = step;
    ctx.status[2] = peer;
    ctx.status[3] = chunk;
    __threadfence();
  }
}

PURLIN_D bool failed(const Context& ctx) { return ldRelaxedGpu32(ctx.status) != 0u; }

// Spin until *flag >= value. Returns false when the time limit ran out or another
// CTA of this call already failed. Called by single threads, not whole CTAs.
PURLIN_D bool waitAtLeast(const Context& ctx, const uint64_t* flag, uint64_t value,
                          uint32_t code, uint32_t step, uint32_t peer, uint32_t chunk) {
  if (ldRelaxedSys(flag) >= value) return ldAcquireSys(flag) >= value;
  const uint64_t start = globalTimerNs();
  uint32_t spins = 0;
  while (ldRelaxedSys(flag) < value) {
    if ((++spins & 63u) == 0u) {
      if (failed(ctx)) return false;
      if (globalTimerNs() - start > ctx.timeoutNs) { fail(ctx, code, step, peer, chunk); return false; }
    }
  }
  return ldAcquireSys(flag) >= value;
}

// True for the last of `expected` arrivals; the counter resets itself for the next use.
PURLIN_D bool lastArrival(uint32_t* counter, uint32_t expected) {
  if (expected <= 1) { __threadfence(); return true; }
  uint32_t old;
  asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  if (old == expected - 1) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(counter), "r"(0u) : "memory");
    return true;
  }
  return false;
}

}  // namespace sig
}  // namespace purlin
