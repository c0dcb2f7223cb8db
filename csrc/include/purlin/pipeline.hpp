// Generic multi-stage prefetch ring: keeps up to Depth asynchronous transfers in flight while earlier ones are used.
//
// Parity: Pipeline<Config>::run of csrc/include/purlin/pipeline.cuh:8-92 in the reference (prime, steady state,
// drain over a shared-memory ring, with the asynchronous mechanism hidden behind a compile-time operation
// interface). The driver below knows nothing about how data moves; the operation supplies:
//
//   void prepare();                         once, before anything else
//   void prefetch(int slot, size_t stage);  start the asynchronous transfer of `stage` into ring slot `slot`
//   void commit();                          close the group of transfers started since the last commit
//   template <int N> void wait();           block until at most N committed groups are still in flight
//   void consume(int slot, size_t stage);   use the data of `stage`, now resident in `slot`
//   void advance();                         once per stage, after consume (pointer bumps, barriers)
//
// Schedule for S stages and depth D: the first min(D, S) stages are prefetched and committed one group each;
// then for every stage s: wait until only the younger groups remain (min(D, S - s) - 1 of them), consume slot
// s % D, refill that slot with stage s + D if there is one, advance. Every stage is prefetched exactly once and
// consumed exactly once, in order; a slot is refilled only after its previous occupant was consumed.
// Works for a whole CTA, for a single warp (several independent pipelines per CTA), and on the host (tests use a
// synchronous operation that records the calls). cp.async, cp.async.bulk with mbarriers, or plain register
// double-buffering all fit the interface; bulk.cuh is the cp.async.bulk instance used by the collectives.
#pragma once
#include <cstddef>

#include "constants.hpp"
#include "static_for.hpp"

namespace purlin {

template <int Depth>
struct Pipeline {
  static_assert(Depth >= 1 && Depth <= 16, "pipeline depth must be in [1, 16]");

  template <class Op>
  PURLIN_HD static void run(Op& op, size_t stages) {
    op.prepare();
    const size_t primed = stages < size_t(Depth) ? stages : size_t(Depth);
    for (size_t s = 0; s < primed; ++s) {
      op.prefetch(int(s), s);
      op.commit();
    }
    for (size_t s = 0; s < stages; ++s) {
      const int slot = int(s % size_t(Depth));
      const size_t left = stages - s;                                   // stages not yet consumed, this one included
      const int inFlight = int(left < size_t(Depth) ? left : size_t(Depth));
      staticSwitch<Depth>(inFlight - 1, [&](auto n) { op.template wait<decltype(n)::value>(); });
      op.consume(slot, s);
      if (s + size_t(Depth) < stages) {
        op.prefetch(slot, s + size_t(Depth));
        op.commit();
      }
      op.advance();
    }
  }
};

}  // namespace purlin
