// The 16-byte latency packet: 8 bytes of payload and an 8-byte flag written by
// one 128-bit store, so the flag can never be seen before its data.
//
// Parity: csrc/include/purlin/packet.cuh:8-88 of the reference (same packet
// format, same relaxed system-scope 128-bit accesses, same multimem broadcast).
// Waits are bounded (see signal.cuh).
#pragma once
#include "signal.cuh"

namespace purlin {

struct alignas(16) Packet {
  uint64_t data;
  uint64_t flag;
};
static_assert(sizeof(Packet) == kPacketBytes, "packet format");

namespace pkt {

PURLIN_D void write(Packet* p, uint64_t data, uint64_t flag) {
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(data), "l"(flag) : "memory");
}
PURLIN_D Packet load(const Packet* p) {
  Packet v;
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.data), "=l"(v.flag) : "l"(p) : "memory");
  return v;
}
// One store, delivered by the NVSwitch to the same offset on every rank.
PURLIN_D void writeMulticast(Packet* mc, uint64_t data, uint64_t flag) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "r"(uint32_t(data)), "r"(uint32_t(data >> 32)), "r"(uint32_t(flag)), "r"(uint32_t(flag >> 32))
               : "memory");
}
// Spin until the packet carries `flag`; false when the time limit ran out.
PURLIN_D bool read(const Context& ctx, const Packet* p, uint64_t flag, uint64_t& data,
                   uint32_t code, uint32_t step, uint32_t peer) {
  Packet v = load(p);
  if (v.flag != flag) {
    const uint64_t start = sig::globalTimerNs();
    uint32_t spins = 0;
    do {
      v = load(p);
      if ((++spins & 63u) == 0u) {
        if (sig::failed(ctx)) return false;
        if (sig::globalTimerNs() - start > ctx.timeoutNs) { sig::fail(ctx, code, step, peer, 0); return false; }
      }
    } while (v.flag != flag);
  }
  data = v.data;
  return true;
}

}  // namespace pkt
}  // namespace purlin
