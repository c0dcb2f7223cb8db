/* C entry points of the tcgen05 GEMM and of the tensor-parallel kernels fused with their collective.
 * No counterpart in the reference (it has no GEMM); see csrc/src/gemm_sm100.cu. */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { PURLIN_EPI_STORE = 0, PURLIN_EPI_SWIGLU = 1 };

/* C[M,N] = A[M,K] * B[N,K]^T, bf16 row-major operands (K contiguous), fp32 accumulation, bf16 output.
 * PURLIN_EPI_SWIGLU: B's rows alternate 16 gate rows and 16 up rows; C is [M, N/2] = silu(gate) * up.
 * bn: tile width (multiple of 16, at most 256); 0 lets the library choose. status: 4 device words or NULL. */
int purlin_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int bn,
                     uint32_t* status, void* stream);

typedef struct PurlinTpContext PurlinTpContext;

/* Bytes of symmetric memory one rank needs for the fused kernels at these maximum shapes:
 * all-gather -> GEMM over activations [M, kAg]; GEMM -> reduce-scatter producing [M, nRs]. */
size_t purlin_tp_workspace_bytes(int world, int M, int kAg, int nRs);
PurlinTpContext* purlin_tp_create(int rank, int world, const uint64_t* peerPtrs, int M, int kAg, int nRs,
                                  uint64_t timeoutNs, void* stream);
int purlin_tp_destroy(PurlinTpContext* ctx, void* stream);
int purlin_tp_status(PurlinTpContext* ctx, uint32_t* out4, void* stream);
int purlin_tp_clear_status(PurlinTpContext* ctx, void* stream);

/* out[M, N or N/2] = epilogue(allgather(xLocal)[M, K] * W[N, K]^T). xLocal is this rank's [M / world, K] rows. */
int purlin_tp_ag_gemm(PurlinTpContext* ctx, const void* xLocal, const void* W, void* out, int M, int N, int K,
                      int epilogue, void* stream);
/* out[M / world, N] = this rank's rows of sum over ranks of (A[M, K] * W[N, K]^T). */
int purlin_tp_gemm_rs(PurlinTpContext* ctx, const void* A, const void* W, void* out, int M, int N, int K, void* stream);

#ifdef __cplusplus
}
#endif
