/* C entry points of libpurlin (loaded by the Python package with ctypes, usable from C).
 *
 * The reference exposes its host API only as C++ templates and a pybind11
 * module generated at run time (purlin/bindings.py:16-453). This build ships a
 * prebuilt shared library instead, so the same calls are plain C symbols:
 * raw device pointers, byte counts, enums as ints, a stream as void*.
 * Every function returns 0 on success; purlin_last_error() explains a failure.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct PurlinHostContext PurlinHostContext;

const char* purlin_last_error(void);
int purlin_version(void);

/* ---- layout engine (no GPU needed) ---- */
size_t purlin_plan_sizeof(void);
size_t purlin_policy_sizeof(void);
/* Fills `ws[8]` = {stagingTRSize, lrOffset, signalOffset, gatherOffset, consumedOffset, varLenOffset, totalBytes, packetStride}. */
int purlin_workspace_layout(int world, size_t stagingTRSize, size_t* ws);
/* Builds the plan of one call. `sizes`/`outSizes` may be NULL for fixed-size collectives.
 * `policy` NULL: the tuning table or the built-in default chooses. `policyOut` (optional) receives the choice. */
int purlin_plan_build(int collective, int world, int rank, size_t bytes, const size_t* sizes, const size_t* outSizes,
                      int dtype, int reduceOp, int mode, int multicastAvailable, int inPlace, size_t stagingTRSize,
                      const void* policy, void* planOut, void* policyOut);
/* Static bounds check of a plan against one rank's buffer extents (every plan the library builds has passed it). */
int purlin_plan_check(const void* plan, int world, size_t stagingTRSize, size_t srcBytes, size_t dstBytes);
int purlin_default_policy(int collective, int world, size_t bytes, int dtype, int mode, int multicastAvailable,
                          size_t stagingTRSize, void* policyOut);
int purlin_topology(int inLayout, int outLayout, int op, int cyclic, int* out8);
int purlin_tuning_clear(void);
int purlin_tuning_add(int collective, int world, uint64_t maxBytes, const void* policy);
size_t purlin_tuning_size(void);

/* ---- CPU interpreter of a plan: `world` ranks in one process over host memory ---- */
int purlin_sim_run(int collective, int world, size_t bytes, const size_t* sizesMatrix, int dtype, int reduceOp, int mode,
                   size_t stagingTRSize, const void* policy, const void* const* srcs, void* const* dsts,
                   int dropRank, uint32_t* statusOut);

/* The same interpreter on a SEQUENCE of calls with no barrier between them: a rank starts its next call as soon as its
 * own steps are done, and a seeded random scheduler moves one agent one chunk at a time. collectives / bytes /
 * sizesMatrices (NULL entries for fixed-size forms): one entry per call; srcs / dsts: nCalls x world pointers, call-major. */
int purlin_sim_run_overlapped(int nCalls, const int* collectives, const size_t* bytes, const size_t* const* sizesMatrices,
                              int world, int dtype, int reduceOp, int mode, size_t stagingTRSize, const void* policy,
                              const void* const* srcs, void* const* dsts, uint64_t seed, int quantum, int multicastAvailable,
                              uint32_t* statusOut);

/* ---- contexts ---- */
/* peerPtrs[world]: base of every rank's symmetric workspace block (peerPtrs[rank] is local).
 * multicastPtr: NVLS alias of the same block, or 0. Honours PURLIN_DISABLE_MULTIMEM and PURLIN_DISABLE_MULTIMEM_LR. */
PurlinHostContext* purlin_context_create(int rank, int world, const uint64_t* peerPtrs, uint64_t multicastPtr,
                                         size_t stagingTRSize, uint64_t timeoutNs, void* stream);
int purlin_context_destroy(PurlinHostContext* ctx, void* stream);
int purlin_context_status(PurlinHostContext* ctx, uint32_t* out4, void* stream);   /* synchronises the stream */
int purlin_context_clear_status(PurlinHostContext* ctx, void* stream);
int purlin_context_set_timeout(PurlinHostContext* ctx, uint64_t timeoutNs);
uint64_t purlin_context_seq(PurlinHostContext* ctx, void* stream);                 /* synchronises the stream */
int purlin_context_has_multicast(PurlinHostContext* ctx);
/* Device-side timing of recent calls (contexts created with PURLIN_TRACE=1): up to maxRecords records of four words
 * {call sequence, start ns, end ns, payload bytes | collective << 56}, oldest first. Returns the count, -1 when off. */
int purlin_context_trace(PurlinHostContext* ctx, uint64_t* out, int maxRecords, void* stream);
const void* purlin_context_device_struct(PurlinHostContext* ctx);                   /* host copy of the device Context */
size_t purlin_context_sizeof(void);

/* ---- collectives: one kernel launch each, no host synchronisation ---- */
int purlin_collective(PurlinHostContext* ctx, int collective, const void* src, void* dst, size_t bytes,
                      const size_t* sizes, const size_t* outSizes, int dtype, int reduceOp, int mode,
                      const void* policy, void* stream);
/* Any fixed-size collective through a short signature: traits = dtype | reduceOp << 8 | mode << 16 (zero for the copy collectives). */
int purlin_call_fixed(PurlinHostContext* ctx, int collective, const void* src, void* dst, size_t bytes, unsigned traits, void* stream);
int purlin_all_reduce(PurlinHostContext* ctx, const void* src, void* dst, size_t bytes, int dtype, int reduceOp, int mode, void* stream);
int purlin_all_gather(PurlinHostContext* ctx, const void* src, void* dst, size_t bytesPerRank, void* stream);
int purlin_all_gather_v(PurlinHostContext* ctx, const void* src, void* dst, const size_t* bytesList, void* stream);
int purlin_reduce_scatter(PurlinHostContext* ctx, const void* src, void* dst, size_t bytesPerRankOut, int dtype, int reduceOp, int mode, void* stream);
int purlin_reduce_scatter_v(PurlinHostContext* ctx, const void* src, void* dst, const size_t* bytesList, int dtype, int reduceOp, int mode, void* stream);
int purlin_all_to_all(PurlinHostContext* ctx, const void* src, void* dst, size_t bytesPerPeer, void* stream);
int purlin_all_to_all_v(PurlinHostContext* ctx, const void* src, void* dst, const size_t* inSplits, const size_t* outSplits, void* stream);

/* ---- single-GPU emulation: `world` virtual ranks run as rows of one cooperative grid ---- */
int purlin_emu_collective(PurlinHostContext* const* ctxs, int world, int collective, const void* const* srcs, void* const* dsts,
                          size_t bytes, const size_t* sizesMatrix, int dtype, int reduceOp, int mode, const void* policy,
                          int absentRank, void* stream);

/* ---- point-to-point copy through the Atom (push or pull over a peer pointer) ---- */
int purlin_p2p_copy(void* dst, const void* src, size_t bytes, int blocks, int threads, void* stream);

/* ---- native symmetric-memory provider on the CUDA virtual-memory API (+ NVLS multicast alias) ----
 * create -> all-gather (pid, fd) -> map_peers; then, if multicast is supported on every rank:
 * rank 0 multicast_create -> broadcast (pid, fd) -> multicast_join everywhere -> barrier -> multicast_bind -> barrier.
 * Release: barrier -> detach everywhere -> barrier -> destroy. */
typedef struct PurlinVmmBlock PurlinVmmBlock;
int purlin_vmm_multicast_supported(int device);
PurlinVmmBlock* purlin_vmm_create(int device, size_t bytes, int rank, int world);
size_t purlin_vmm_bytes(const PurlinVmmBlock* block);
int purlin_vmm_local_handle(const PurlinVmmBlock* block, int* pid, int* fd);
int purlin_vmm_map_peers(PurlinVmmBlock* block, const int* pids, const int* fds);
uint64_t purlin_vmm_peer_ptr(const PurlinVmmBlock* block, int rank);
int purlin_vmm_multicast_create(PurlinVmmBlock* block, int* pid, int* fd);
int purlin_vmm_multicast_join(PurlinVmmBlock* block, int pid, int fd);
int purlin_vmm_multicast_bind(PurlinVmmBlock* block);
uint64_t purlin_vmm_multicast_ptr(const PurlinVmmBlock* block);
int purlin_vmm_exchange_done(void);   /* after the barrier that follows mapping: peers may no longer duplicate this process's descriptors */
int purlin_vmm_detach(PurlinVmmBlock* block);
int purlin_vmm_destroy(PurlinVmmBlock* block);

#ifdef __cplusplus
}
#endif
