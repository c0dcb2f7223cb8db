/* C entry points of the expert-parallel MoE token exchange (csrc/src/moe.cu). No counterpart in the reference. */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct PurlinMoeContext PurlinMoeContext;

/* Symmetric bytes per rank: receive buffer + expert-output buffer of capacityRows rows each, count matrix, flags. */
size_t purlin_moe_workspace_bytes(int world, int capacityRows, int hidden, int experts);
PurlinMoeContext* purlin_moe_create(int rank, int world, const uint64_t* peerPtrs, int maxTokens, int hidden, int experts,
                                    int topk, int capacityRows, uint64_t timeoutNs, void* stream);
int purlin_moe_destroy(PurlinMoeContext* ctx, void* stream);
int purlin_moe_status(PurlinMoeContext* ctx, uint32_t* out4, void* stream);
int purlin_moe_clear_status(PurlinMoeContext* ctx, void* stream);
void* purlin_moe_recv_buffer(PurlinMoeContext* ctx);   /* [capacityRows, hidden] bf16, expert-major after dispatch */
void* purlin_moe_out_buffer(PurlinMoeContext* ctx);    /* [capacityRows, hidden] bf16, written by the experts, read by combine */

/* softmax over logits [tokens, experts] (fp32), top-k; slot = position of each choice among this rank's rows of that expert */
int purlin_moe_route(PurlinMoeContext* ctx, const float* logits, int tokens, int normalize, int32_t* topkIdx, float* topkWeight,
                     int32_t* slot, void* stream);
/* x [tokens, hidden] bf16 -> every chosen expert's GPU, already in expert-major order. sentRow [tokens, topk] and
 * recvCounts [experts / world + 1] (rows per local expert, then their total) are outputs. dispatch and combine alternate. */
int purlin_moe_dispatch(PurlinMoeContext* ctx, const void* x, int tokens, const int32_t* topkIdx, const int32_t* slot,
                        int32_t* sentRow, int32_t* recvCounts, int blocks, void* stream);
/* y [tokens, hidden] = sum over k of topkWeight * (row sentRow of the expert-output buffer on that expert's GPU) */
int purlin_moe_combine(PurlinMoeContext* ctx, void* y, int tokens, const int32_t* topkIdx, const float* topkWeight,
                       const int32_t* sentRow, int blocks, void* stream);

#ifdef __cplusplus
}
#endif
