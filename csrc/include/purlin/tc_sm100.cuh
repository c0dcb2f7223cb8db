// Thin inline-PTX layer over the Blackwell tensor-core pipeline: mbarriers, TMA tile
// loads (never with cluster multicast), TMEM allocation, tcgen05.mma / commit / ld.
//
// No counterpart in the reference (it contains no tensor-core code at all). Every
// wait on an mbarrier is bounded: when the time limit runs out the waiter raises the
// CTA's abort word, records a status and the kernel unwinds, frees its TMEM and returns.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "constants.hpp"
#include "signal.cuh"

namespace purlin {
namespace tc {

PURLIN_D uint32_t smemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---- mbarrier ----
PURLIN_D void mbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
PURLIN_D void mbarFenceInit() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
PURLIN_D void mbarExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
PURLIN_D void mbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
PURLIN_D bool mbarTryWait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  // cluster-scope acquire: the arrival may come from the other CTA of a pair
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait. `abortWord` is a CTA-shared int: non-zero means some role gave up.
PURLIN_D bool mbarWait(uint32_t bar, uint32_t parity, volatile int* abortWord, uint64_t timeoutNs) {
  if (mbarTryWait(bar, parity)) return true;
  const uint64_t start = sig::globalTimerNs();
  uint32_t spins = 0;
  while (!mbarTryWait(bar, parity)) {
    if ((++spins & 31u) == 0u) {
      if (*abortWord) return false;
      if (sig::globalTimerNs() - start > timeoutNs) { *abortWord = 1; return false; }
    }
  }
  return true;
}

// ---- TMA (tile mode, this CTA only) ----
PURLIN_D void tmaLoad2d(uint32_t smemDst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smemDst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Hint: bring a tile into L2 (no shared-memory destination, nothing to wait for). Issued several k-blocks ahead of the
// real load it turns a DRAM miss on the critical path into an L2 hit.
PURLIN_D void tmaPrefetchL2(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
PURLIN_D void tmaPrefetchDescriptor(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
PURLIN_D void fenceProxyAsync() { asm volatile("fence.proxy.async;" ::: "memory"); }
// Tile store: shared memory (this CTA) -> global memory, tracked by the issuing thread's bulk async-groups. Out-of-range
// parts of the box are clipped. Writers of the shared-memory tile run fenceProxyAsyncShared() before the issuing thread
// is told (their generic-proxy stores must be visible to the async proxy).
PURLIN_D void fenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
PURLIN_D void tmaStore2d(const CUtensorMap* map, int x, int y, uint32_t smemSrc) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smemSrc), "r"(x), "r"(y) : "memory");
}
PURLIN_D void bulkCommitGroup() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most N of this thread's groups may still be READING their shared-memory source
template <int N> PURLIN_D void bulkWaitGroupRead() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// at most N of this thread's groups may still be in flight at all (their global writes included)
template <int N> PURLIN_D void bulkWaitGroup() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

// ---- CTA pairs (cluster of two): the pair shares one 256-row MMA; CTA 0 issues it ----
PURLIN_D uint32_t clusterCtaRank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
// address of the same shared-memory offset inside CTA `rank` of the cluster
PURLIN_D uint32_t mapToCta(uint32_t smemAddress, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smemAddress), "r"(rank));
  return out;
}
PURLIN_D void clusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
PURLIN_D void mbarArriveCluster(uint32_t clusterBarAddress) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterBarAddress) : "memory");
}
// tile load of one CTA of a pair; the transaction bytes are credited to a barrier that may live in the other CTA
PURLIN_D void tmaLoad2dPair(uint32_t smemDst, const CUtensorMap* map, int x, int y, uint32_t clusterBarAddress) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smemDst), "l"(map), "r"(clusterBarAddress), "r"(x), "r"(y) : "memory");
}
PURLIN_D void tmemAllocPair(uint32_t smemResult, uint32_t columns) {   // one whole warp in each CTA of the pair
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemResult), "r"(columns) : "memory");
}
PURLIN_D void tmemRelinquishPair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
PURLIN_D void tmemDeallocPair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// 256 x n x 16 MMA across the pair: each CTA supplies its 128 rows of A and its half of B's columns
PURLIN_D void mmaPair(uint32_t tmemD, uint64_t aDesc, uint64_t bDesc, uint32_t iDesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmemD), "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate) : "memory");
}
PURLIN_D void mmaCommitPair(uint32_t clusterBarAddress) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(clusterBarAddress) : "memory");
}

// ---- TMEM ----
PURLIN_D void tmemAlloc(uint32_t smemResult, uint32_t columns) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemResult), "r"(columns) : "memory");
}
PURLIN_D void tmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
PURLIN_D void tmemDealloc(uint32_t taddr, uint32_t columns) {     // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
PURLIN_D void fenceBeforeThreadSync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
PURLIN_D void fenceAfterThreadSync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ----
// K-major operand tile in shared memory, 128-byte swizzle: rows of 64 bf16 (128 B), groups of 8 rows
// form a 1024-byte swizzle atom. Start address in 16-byte units, leading offset 1 (unused for swizzled
// K-major), stride offset 1024 B between 8-row groups, descriptor version 1, layout SWIZZLE_128B (2).
PURLIN_D uint64_t smemDescSw128(uint32_t smemByteAddr) {
  const uint32_t lo = ((smemByteAddr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return uint64_t(lo) | (uint64_t(hi) << 32);
}
// bf16 x bf16 -> fp32, both operands K-major, M = 128 (one CTA) or 256 (a CTA pair), N = n (multiple of 16, at most 256).
PURLIN_D uint32_t instrDescBf16(uint32_t n, uint32_t m = 128u) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- MMA ----
PURLIN_D void mma(uint32_t tmemD, uint64_t aDesc, uint64_t bDesc, uint32_t iDesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmemD), "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate) : "memory");
}
// arrives on the mbarrier when every MMA issued so far by this thread has completed
PURLIN_D void mmaCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 columns of fp32: thread `lane` receives row (laneBase + lane), columns [col, col + 32)
PURLIN_D void tmemLoad32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
PURLIN_D void tmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, tied to the registers of an earlier tmemLoad32: when other work sits between a load and its wait
// (software pipelining), the compiler must not move a use of those registers above the wait.
PURLIN_D void tmemLoadWaitFor(uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
        "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
        "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
        "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :: "memory");
}

}  // namespace tc
}  // namespace purlin
