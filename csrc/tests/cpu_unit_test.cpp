// Host-only unit tests of the compile-time loop and the prefetch-ring driver (no GPU, no CUDA headers).
//
// Counterpart of csrc/tests/static_for.cu:6-77 and csrc/tests/pipeline.cu:8-156 in the reference: the loop's
// order, index type, empty-loop and non-copyable-functor behaviour; the pipeline's hook order and data for depths
// 1/2/4/8 and stage counts 0, 1, depth, depth+1 and 3*depth+2, driven by a fake operation whose "asynchronous"
// transfers complete only when wait<N>() says they may, so a consume that runs too early reads a poisoned slot.
// The same headers compile for the device; device_api_test.cu runs them inside a kernel.
#include <cstdio>
#include <memory>
#include <string>
#include <type_traits>
#include <vector>

#include "purlin/pipeline.hpp"
#include "purlin/plan.hpp"
#include "purlin/static_for.hpp"

using namespace purlin;

static int g_failures = 0;
#define CHECK(cond, what)                                                                        \
  do {                                                                                           \
    if (cond) std::printf("ok    %s\n", what);                                                  \
    else { std::printf("FAIL  %s (%s:%d)\n", what, __FILE__, __LINE__); ++g_failures; }          \
  } while (0)

// ---- staticFor ----
constexpr int sumTo() {
  int t = 0;
  staticFor<5>([&](auto i) { t += decltype(i)::value; });
  return t;
}
static_assert(sumTo() == 10, "staticFor is usable in constant expressions");

struct NeverCalled {
  template <class I> void operator()(I) const { static_assert(sizeof(I) == 0, "an empty loop must not instantiate its body"); }
};

struct MoveOnly {
  std::unique_ptr<int> count = std::make_unique<int>(0);
  template <class I> void operator()(I) { *count += 1; }
};

template <int N> struct Tag { static constexpr int value = N; };

static void testStaticFor() {
  std::vector<int> order;
  staticFor<6>([&](auto i) { order.push_back(decltype(i)::value); });
  CHECK((order == std::vector<int>{0, 1, 2, 3, 4, 5}), "staticFor visits 0..N-1 in order");
  staticFor<0>(NeverCalled{});
  CHECK(true, "staticFor<0> does not instantiate its body");
  MoveOnly m;
  staticFor<4>(m);
  CHECK(*m.count == 4, "staticFor takes a non-copyable functor by reference");
  bool isConstant = false;
  staticFor<1>([&](auto i) { isConstant = std::is_same_v<decltype(i), std::integral_constant<int, 0>>; });
  CHECK(isConstant, "the index is std::integral_constant<int, I>");
  int picked = -1;
  staticFor<3>([&](auto i) { if (Tag<decltype(i)::value>::value == 2) picked = i; });
  CHECK(picked == 2, "the index selects template arguments and converts to int");
  int seen = -1;
  CHECK(staticSwitch<4>(3, [&](auto i) { seen = decltype(i)::value; }) && seen == 3, "staticSwitch maps a run-time value to a constant");
  CHECK(!staticSwitch<4>(4, [&](auto) { seen = 99; }) && seen == 3, "staticSwitch reports a value outside the range");
}

// ---- Pipeline with a fake asynchronous operation ----
template <int Depth>
struct FakeOp {
  std::vector<int> source;            // stage -> payload
  int ring[Depth];                    // what a consumer would read
  struct Pending { int slot; int value; };
  std::vector<std::vector<Pending>> groups;   // committed groups, oldest first
  std::vector<Pending> open;                  // transfers since the last commit
  std::vector<std::string> log;
  std::vector<int> consumed;
  int prepares = 0, prefetches = 0, commits = 0, waits = 0, advances = 0, badWaits = 0, earlyReads = 0, maxInFlight = 0;

  explicit FakeOp(size_t stages) {
    for (size_t s = 0; s < stages; ++s) source.push_back(1000 + int(s) * 7);
    for (int& r : ring) r = -1;
  }
  void prepare() { ++prepares; log.push_back("prepare"); }
  void prefetch(int slot, size_t stage) {
    ++prefetches;
    if (slot < 0 || slot >= Depth || slot != int(stage % Depth)) ++badWaits;
    ring[slot] = -1;                                   // the slot is being overwritten: poisoned until the transfer lands
    open.push_back({slot, source[stage]});
    log.push_back("prefetch " + std::to_string(stage));
  }
  void commit() {
    ++commits;
    groups.push_back(open);
    open.clear();
    if (int(groups.size()) > maxInFlight) maxInFlight = int(groups.size());
    log.push_back("commit");
  }
  template <int N> void wait() {
    ++waits;
    static_assert(N >= 0 && N < Depth, "wait<N> must leave fewer than Depth groups in flight");
    if (int(groups.size()) < N) ++badWaits;            // asked to leave more in flight than exist
    while (int(groups.size()) > N) {                   // the oldest groups land
      for (const Pending& p : groups.front()) ring[p.slot] = p.value;
      groups.erase(groups.begin());
    }
    log.push_back("wait " + std::to_string(N));
  }
  void consume(int slot, size_t stage) {
    if (ring[slot] != source[stage]) ++earlyReads;
    consumed.push_back(ring[slot]);
    log.push_back("consume " + std::to_string(stage));
  }
  void advance() { ++advances; log.push_back("advance"); }
};

template <int Depth>
static void testPipelineDepth() {
  const size_t counts[] = {0, 1, size_t(Depth), size_t(Depth) + 1, 3 * size_t(Depth) + 2};
  bool ok = true;
  for (size_t stages : counts) {
    FakeOp<Depth> op(stages);
    Pipeline<Depth>::run(op, stages);
    ok = ok && op.prepares == 1 && op.prefetches == int(stages) && op.commits == int(stages) && op.waits == int(stages) &&
         op.advances == int(stages) && op.badWaits == 0 && op.earlyReads == 0 && op.consumed == op.source && op.groups.empty() &&
         op.open.empty() && op.maxInFlight <= Depth && (stages < size_t(Depth) || op.maxInFlight == Depth || stages == 0);
    if (!ok) { std::printf("      depth %d stages %zu: prefetches %d commits %d waits %d badWaits %d earlyReads %d maxInFlight %d\n", Depth, stages,
                           op.prefetches, op.commits, op.waits, op.badWaits, op.earlyReads, op.maxInFlight); break; }
  }
  const std::string what = "pipeline depth " + std::to_string(Depth) + ": every stage prefetched once, consumed once, in order, never early";
  CHECK(ok, what.c_str());
}

static void testPipelineOrder() {
  FakeOp<2> op(3);
  Pipeline<2>::run(op, 3);
  const std::vector<std::string> want = {"prepare", "prefetch 0", "commit", "prefetch 1", "commit",
                                         "wait 1", "consume 0", "prefetch 2", "commit", "advance",
                                         "wait 1", "consume 1", "advance",
                                         "wait 0", "consume 2", "advance"};
  CHECK(op.log == want, "pipeline hook order for depth 2, three stages (prime, steady state, drain)");
  // two independent pipelines (one per warp in a kernel) do not share state
  FakeOp<4> a(9), b(5);
  Pipeline<4>::run(a, 9);
  Pipeline<4>::run(b, 5);
  CHECK(a.consumed == a.source && b.consumed == b.source && a.earlyReads + b.earlyReads == 0, "independent pipelines keep separate rings");
}

// ---- aligned partitioning (used by every CTA to find its slice) ----
static void testPartition() {
  bool ok = true;
  for (size_t bytes : {size_t(0), size_t(32), size_t(96), size_t(4096), size_t(1000000) / 32 * 32, size_t(3) << 20}) {
    for (int parts : {1, 2, 3, 7, 16, 148}) {
      size_t at = 0;
      size_t biggest = 0, smallest = ~size_t(0);
      for (int p = 0; p < parts; ++p) {
        const Span s = partitionAligned(bytes, parts, p, kAccessAlign);
        ok = ok && s.offset == at && s.bytes % kAccessAlign == 0;
        at += s.bytes;
        biggest = s.bytes > biggest ? s.bytes : biggest;
        smallest = s.bytes < smallest ? s.bytes : smallest;
      }
      ok = ok && at == bytes && biggest - smallest <= size_t(kAccessAlign);
    }
  }
  CHECK(ok, "partitionAligned: contiguous, aligned, complete, balanced within one access");
}

int main() {
  testStaticFor();
  testPipelineDepth<1>();
  testPipelineDepth<2>();
  testPipelineDepth<4>();
  testPipelineDepth<8>();
  testPipelineOrder();
  testPartition();
  std::printf("%s: %d failure(s)\n", g_failures ? "FAILED" : "PASSED", g_failures);
  return g_failures ? 1 : 0;
}
