// Split policies for variable-length collectives: how a total is divided among ranks (or among the streams of an
// all-to-all) in benchmarks and stress tests.
//
// Behavioural counterpart of csrc/support/purlin/benchmark/variable_counts.cuh in the reference (Zipf splits with a
// power-of-two unit and largest-remainder apportionment; exponents 0, 1/8, 1/4, 1/2, 1) and of the skew generators in
// csrc/tests/{agvskew,rsvskew,a2avskew}.cu (seeded skew of 0/25/50 %, sparse traffic, hot ring). All outputs are
// multiples of the unit, sum exactly to the total, and depend only on the arguments (no floating-point library
// calls beyond sqrt, which IEEE-754 rounds identically everywhere), so every rank derives the same lists without
// communicating.
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <numeric>
#include <string>
#include <vector>

namespace purlin { void setError(const std::string& e); }

namespace {

constexpr size_t kSplitAlign = 128;

// largest power-of-two unit (>= 128 B) dividing `total` that still leaves eight units per rank
bool splitUnit(size_t total, int world, size_t& unit) {
  if (world <= 0 || world > 32) { purlin::setError("split world size must be in [1, 32]"); return false; }
  if (total == 0 || total % kSplitAlign) { purlin::setError("split total must be a positive multiple of 128 bytes"); return false; }
  unit = kSplitAlign;
  while (total % (unit * 2) == 0 && total / (unit * 2) >= size_t(8) * size_t(world)) unit *= 2;
  return true;
}

// splitmix64: a tiny seeded generator with a fixed, documented sequence
uint64_t mix(uint64_t& s) {
  uint64_t z = (s += 0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

// units[i] = floor(quota_i), then the leftover units go to the largest fractional parts (ties: lowest index)
void largestRemainder(const std::vector<long double>& weight, size_t units, std::vector<size_t>& out) {
  const size_t n = weight.size();
  long double sum = 0;
  for (long double w : weight) sum += w;
  out.assign(n, 0);
  std::vector<long double> frac(n, 0);
  size_t given = 0;
  for (size_t i = 0; i < n; ++i) {
    const long double q = sum > 0 ? (long double)units * weight[i] / sum : 0;
    out[i] = size_t(std::floor(q));
    frac[i] = q - std::floor(q);
    given += out[i];
  }
  std::vector<size_t> order(n);
  std::iota(order.begin(), order.end(), size_t(0));
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return frac[a] > frac[b]; });
  for (size_t k = 0; given < units; ++k, ++given) ++out[order[k % n]];
}

}  // namespace

extern "C" {

size_t purlin_split_unit(size_t total, int world) {
  size_t unit = 0;
  return splitUnit(total, world, unit) ? unit : 0;
}

// Zipf: rank r receives units in proportion to 1 / (r + 1)^(eighths / 8); eighths in {0, 1, 2, 4, 8}.
int purlin_zipf_splits(size_t total, int world, int eighths, size_t* out) {
  size_t unit = 0;
  if (!splitUnit(total, world, unit)) return 1;
  if (eighths != 0 && eighths != 1 && eighths != 2 && eighths != 4 && eighths != 8) { purlin::setError("Zipf exponent must be 0, 0.125, 0.25, 0.5 or 1"); return 1; }
  const size_t units = total / unit;
  std::vector<size_t> u;
  if (eighths == 8) {
    // exact integer weights lcm(1..world) / (r + 1)
    uint64_t scale = 1;
    for (int r = 1; r <= world; ++r) scale = std::lcm(scale, uint64_t(r));
    std::vector<uint64_t> w(world);
    uint64_t wsum = 0;
    for (int r = 0; r < world; ++r) { w[r] = scale / uint64_t(r + 1); wsum += w[r]; }
    if (units > UINT64_MAX / w[0]) { purlin::setError("split total too large for this world size"); return 1; }
    u.assign(world, 0);
    std::vector<uint64_t> rem(world);
    size_t given = 0;
    for (int r = 0; r < world; ++r) { const uint64_t num = uint64_t(units) * w[r]; u[r] = size_t(num / wsum); rem[r] = num % wsum; given += u[r]; }
    std::vector<int> order(world);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return rem[a] > rem[b]; });
    for (int k = 0; given < units; ++k, ++given) ++u[order[k % world]];
  } else {
    if (units > (size_t(1) << 32)) { purlin::setError("split total too large for a fractional Zipf exponent"); return 1; }
    std::vector<long double> w(world);
    for (int r = 0; r < world; ++r) {
      double root = double(r + 1);
      for (int e = eighths; e > 0 && e < 8; e *= 2) root = std::sqrt(root);   // each square root halves the exponent
      w[r] = eighths == 0 ? 1.0L : 1.0L / (long double)root;
    }
    largestRemainder(w, units, u);
  }
  for (int r = 0; r < world; ++r) out[r] = u[r] * unit;
  return 0;
}

// Seeded skew: `percent` of the total is moved from an even split to one seeded "heavy" rank, the rest stays even.
int purlin_skew_splits(size_t total, int world, int percent, uint64_t seed, size_t* out) {
  size_t unit = 0;
  if (!splitUnit(total, world, unit)) return 1;
  if (percent < 0 || percent > 100) { purlin::setError("skew must be 0..100 percent"); return 1; }
  const size_t units = total / unit;
  uint64_t s = seed;
  const int heavy = int(mix(s) % uint64_t(world));
  const size_t moved = units * size_t(percent) / 100;
  std::vector<long double> even(world, 1.0L);
  std::vector<size_t> u;
  largestRemainder(even, units - moved, u);
  u[heavy] += moved;
  for (int r = 0; r < world; ++r) out[r] = u[r] * unit;
  return 0;
}

// All-to-all-v traffic matrices, row r = what rank r sends. All entries are multiples of 128 bytes.
// sparse: only `active` seeded (source, destination) pairs per source carry `bytes`; the rest are empty.
int purlin_sparse_matrix(int world, int active, size_t bytes, uint64_t seed, size_t* out) {
  if (world <= 0 || world > 32 || active < 0 || active > world || bytes % kSplitAlign) { purlin::setError("invalid sparse matrix arguments"); return 1; }
  uint64_t s = seed;
  for (int r = 0; r < world; ++r) {
    std::vector<int> dst(world);
    std::iota(dst.begin(), dst.end(), 0);
    for (int i = world - 1; i > 0; --i) std::swap(dst[i], dst[int(mix(s) % uint64_t(i + 1))]);
    for (int d = 0; d < world; ++d) out[size_t(r) * world + d] = 0;
    for (int k = 0; k < active; ++k) out[size_t(r) * world + dst[k]] = bytes;
  }
  return 0;
}
// hot ring: `percent` of every rank's bytes go to the next rank, the rest is spread evenly over the others.
int purlin_hotring_matrix(int world, size_t bytesPerRank, int percent, size_t* out) {
  if (world <= 1 || world > 32 || bytesPerRank % kSplitAlign || percent < 0 || percent > 100) { purlin::setError("invalid hot-ring arguments"); return 1; }
  const size_t units = bytesPerRank / kSplitAlign, hot = units * size_t(percent) / 100;
  for (int r = 0; r < world; ++r) {
    std::vector<long double> even(world - 1, 1.0L);
    std::vector<size_t> rest;
    largestRemainder(even, units - hot, rest);
    int k = 0;
    for (int d = 0; d < world; ++d) {
      if (d == (r + 1) % world) { out[size_t(r) * world + d] = hot * kSplitAlign; continue; }
      out[size_t(r) * world + d] = rest[k++ % (world - 1)] * kSplitAlign;
    }
    // the self slot took one share of `rest`; that is intended: local traffic stays in the pattern
  }
  return 0;
}

}  // extern "C"
