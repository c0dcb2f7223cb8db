// Compile-time limits and the byte geometry of the symmetric workspace.
//
// Parity: csrc/include/purlin/constants.cuh:8-24 of the reference (same limits:
// 16 ranks per NVLink domain, 8 MiB packet epoch, 256 MiB staging ceiling,
// 1024 chunks), restated for a Blackwell-only build: the access alignment is
// always 32 bytes because every sm_100a global access may be 256 bits wide.
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define PURLIN_HD __host__ __device__
#define PURLIN_D __device__ __forceinline__
#else
#define PURLIN_HD
#define PURLIN_D inline
#endif

namespace purlin {

constexpr int kWarpSize = 32;
constexpr int kMaxRanks = 16;                       // one NVLink scale-up domain
constexpr size_t kAccessAlign = 32;                 // bytes; buffers and byte counts are multiples of this
constexpr size_t kPacketBytes = 16;                 // {u64 data, u64 flag}
constexpr size_t kPacketEpochBytes = 8ull << 20;    // one half of the latency (packet) buffer
constexpr size_t kMinChunkBytes = 256ull << 10;
constexpr size_t kMaxStagingBytes = 256ull << 20;   // one half of the throughput staging buffer
constexpr size_t kDefaultStagingBytes = 256ull << 20;
constexpr int kMaxChunks = 1024;                    // flag values reserved per stream per call
constexpr int kMaxCtas = 148;                       // one per B200 SM
constexpr int kMaxSteps = 56;                       // steps in one plan (stage + local + consume + gather)
constexpr int kCounterSlots = kMaxSteps * kMaxChunks;
constexpr int kSeqWords = 256;                     // copies of the call sequence number: CTA b reads word b % kSeqWords

// Flag value of chunk `k` (0-based) of call number `seq`. Values grow with
// every call and every chunk, so flags are never cleared; waits compare >=.
constexpr int kTraceSlots = 256;   // calls kept by the optional device-side timing ring
constexpr int kSeqShift = 20;
PURLIN_HD constexpr uint64_t flagValue(uint64_t seq, uint64_t chunk) {
  return (seq << kSeqShift) + chunk + 1;
}

PURLIN_HD constexpr size_t roundUp(size_t v, size_t a) { return (v + a - 1) / a * a; }
PURLIN_HD constexpr size_t roundDown(size_t v, size_t a) { return v / a * a; }
PURLIN_HD constexpr size_t ceilDiv(size_t v, size_t a) { return (v + a - 1) / a; }

// Status codes written by bounded device waits (0 = healthy).
enum Status : uint32_t {
  kStatusOk = 0,
  kStatusTimeoutSignal = 1,    // a put/gather/consumed flag never reached its value
  kStatusTimeoutPacket = 2,    // a latency packet never arrived
  kStatusTimeoutArrival = 3,   // a variable-length arrival packet never arrived
  kStatusTimeoutTile = 4,      // a fused-kernel tile flag never arrived
  kStatusTimeoutBarrier = 5,   // an mbarrier phase inside a fused kernel never completed
  kStatusBadPlan = 6,
};

}  // namespace purlin
