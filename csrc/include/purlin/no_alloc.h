/* Allocation-free MoE routing entry point.
 *
 * This entry point has no counterpart in the reference.
 *
 * Who needs it: code that is not allowed to call cudaMalloc at the moment it runs. An inference server that has
 * handed all device memory to its own pool after warm-up, a plugin whose enqueue callback must not allocate, or a
 * process that wants no hidden device synchronisation (cudaMalloc and cudaFree synchronise the device) cannot create
 * a PurlinMoeContext just to route tokens. Here the only scratch memory the routing kernel needs, one counter per
 * expert, lives in a static device array inside the library: 512 counters = 2 KiB, held by every GPU that loads the
 * library until the process exits. The caller passes nothing but inputs and outputs.
 *
 * Rules of use:
 *   - experts must be 32, 64, 128, 256 or 512 (PURLIN_NOALLOC_MAX_EXPERTS); topk 1..8. Anything else is refused
 *     with an error (purlin_last_error()), not truncated.
 *   - The first call on each device resolves the device address of the scratch array (cudaGetSymbolAddress) with that
 *     device current. Make that first call before any stream capture begins.
 *   - Every call on a device shares the same counters. The call clears them on `stream` before the kernel runs, so
 *     consecutive calls on one stream are independent; two calls that can overlap on the GPU (different streams, no
 *     ordering between them) race on the counters and must not be issued.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, on the first call or later.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PURLIN_NOALLOC_MAX_EXPERTS 512

/* softmax over logits [tokens, experts] (fp32), top-k, slot assignment; same results as purlin_moe_route.
 * topkIdx [tokens, topk] int32, topkWeight [tokens, topk] fp32, slot [tokens, topk] int32 are device outputs.
 * Returns 0 on success. */
int purlin_moe_route_noalloc(const float* logits, int tokens, int experts, int topk, int normalize,
                             int32_t* topkIdx, float* topkWeight, int32_t* slot, void* stream);

#ifdef __cplusplus
}
#endif
