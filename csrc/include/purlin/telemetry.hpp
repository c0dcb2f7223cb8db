// NVTX range around every host entry point that launches a kernel.
//
// Parity: PurlinRange of csrc/include/purlin/host/telemetry.cuh:5-8 in the reference (an NVTX3 scoped range in the
// domain "Purlin" with the byte count as payload, compiled in when PURLIN_NVTX=1). The same domain and payload
// convention is used here, for the collectives and also for the fused GEMM, MoE and zero-copy entry points the
// reference does not have, so a timeline shows every launch of this library under one domain.
#pragma once
#include <cstddef>

#if defined(PURLIN_NVTX) && PURLIN_NVTX
#include <nvtx3/nvToolsExt.h>

namespace purlin {

struct NvtxRange {
  NvtxRange(const char* name, size_t bytes) {
    nvtxEventAttributes_t a{};
    a.version = NVTX_VERSION; a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
    a.messageType = NVTX_MESSAGE_TYPE_ASCII; a.message.ascii = name;
    a.payloadType = NVTX_PAYLOAD_TYPE_UNSIGNED_INT64; a.payload.ullValue = bytes;
    static nvtxDomainHandle_t domain = nvtxDomainCreateA("Purlin");
    domain_ = domain;
    nvtxDomainRangePushEx(domain_, &a);
  }
  ~NvtxRange() { nvtxDomainRangePop(domain_); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
 private:
  nvtxDomainHandle_t domain_;
};

}  // namespace purlin
#else
namespace purlin {
struct NvtxRange { NvtxRange(const char*, size_t) {} };
}  // namespace purlin
#endif
