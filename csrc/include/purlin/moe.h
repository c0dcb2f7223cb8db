/* C entry points of the expert-parallel MoE token exchange (csrc/src/moe.cu). No counterpart in the reference.
 *
 * One layer is: route (or plan) -> dispatch -> the experts work on the receive buffer and write the output buffer ->
 * combine. CONTRACT: on every rank, dispatch and combine of one context alternate on one stream (dispatch, combine,
 * dispatch, ...). The kernels reuse the staging and combine buffers of the previous layer without a further
 * handshake; what makes that safe is that a rank writes into a peer's buffers only after it has seen the peer's
 * counts of the same dispatch, which the peer publishes after its previous combine has finished. A call out of order
 * is not run: the kernel reports it through the status word (purlin_moe_status: code 6, where 9 or 10).
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct PurlinMoeContext PurlinMoeContext;

/* Symmetric bytes per rank: a staging area and a combine buffer of world x maxTokens rows each (a token crosses NVLink
 * once per destination GPU), the expert-major receive buffer and the expert-output buffer of capacityRows rows each,
 * the records of the staged rows, the count matrix and the flags. */
size_t purlin_moe_workspace_bytes(int world, int maxTokens, int capacityRows, int hidden, int experts);
PurlinMoeContext* purlin_moe_create(int rank, int world, const uint64_t* peerPtrs, int maxTokens, int hidden, int experts,
                                    int topk, int capacityRows, uint64_t timeoutNs, void* stream);
int purlin_moe_destroy(PurlinMoeContext* ctx, void* stream);
int purlin_moe_status(PurlinMoeContext* ctx, uint32_t* out4, void* stream);
int purlin_moe_clear_status(PurlinMoeContext* ctx, void* stream);
/* Diagnostics (contexts created with PURLIN_MOE_TIMING=1): nanoseconds from the first CTA's start to {last sender end, last
 * receiver end, first sender end, 0} of the dispatches and {last pusher end, last finisher end, first pusher end, 0} of the
 * combines since the previous call of this function. Synchronises the stream. */
int purlin_moe_timing(PurlinMoeContext* ctx, uint64_t* out8, void* stream);
void* purlin_moe_recv_buffer(PurlinMoeContext* ctx);   /* [capacityRows, hidden] bf16, expert-major after dispatch */
void* purlin_moe_out_buffer(PurlinMoeContext* ctx);    /* [capacityRows, hidden] bf16, written by the experts, read by combine */

/* softmax over logits [tokens, experts] (fp32), top-k (total for any input: see moe_route.cuh), then the plan below.
 * topkIdx / topkWeight / slot [tokens, topk] are device outputs the context keeps using until the next route or plan. */
int purlin_moe_route(PurlinMoeContext* ctx, const float* logits, int tokens, int normalize, int32_t* topkIdx, float* topkWeight,
                     int32_t* slot, void* stream);
/* The plan alone, for routing the caller computed itself: slot = position of each (token, expert) pair among this rank's
 * rows of that expert; internally one send-list position per (token, destination GPU). Expert ids outside
 * [0, experts) are reported through the status word and their pairs dropped. */
int purlin_moe_plan(PurlinMoeContext* ctx, const int32_t* topkIdx, const float* topkWeight, int tokens, int32_t* slot, void* stream);
/* x [tokens, hidden] bf16 -> every chosen expert's GPU, in expert-major order in its receive buffer. topkIdx and slot are
 * the arrays of the last route / plan. sentRow [tokens, topk] (optional, may be null: the row of each pair inside its
 * expert GPU's receive buffer) and recvCounts [experts / world + 1] (rows per local expert, then their total) are
 * outputs. `blocks` > 0 sets how many CTAs send (the rest of the grid receives); 0 picks a default. */
int purlin_moe_dispatch(PurlinMoeContext* ctx, const void* x, int tokens, const int32_t* topkIdx, const int32_t* slot,
                        int32_t* sentRow, int32_t* recvCounts, int blocks, void* stream);
/* y [tokens, hidden] = sum over the token's experts of gate weight x expert output row. The weights travelled with the
 * rows at dispatch; topkWeight and sentRow are accepted for symmetry and not read. */
int purlin_moe_combine(PurlinMoeContext* ctx, void* y, int tokens, const int32_t* topkIdx, const float* topkWeight,
                       const int32_t* sentRow, int blocks, void* stream);

#ifdef __cplusplus
}
#endif
