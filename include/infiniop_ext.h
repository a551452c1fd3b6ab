/*
 * infiniop_ext.h - additive entry points of the B200 backend that have no
 * counterpart in the reference library.  Nothing here changes the behaviour of
 * the reference-shaped ABI in infiniop.h.
 */
#ifndef INFINIOP_B200_EXT_H
#define INFINIOP_B200_EXT_H

#include "infiniop.h"

/*
 * Kernel-family switch for tests and benchmarks (no counterpart in the
 * reference).  Several operators have two kernel families, chosen per call
 * from shapes and alignment; this forces one of them process-wide so that both
 * can be held to the same oracle on the same inputs.  variant 0 restores the
 * library's own choice.
 *   family 0 (RoPE):          1 = the strided kernel instead of the bulk-copy pipeline, 2 = the pipeline with bulk
 *                             stores out of shared memory instead of the threads' own stores
 *   family 1 (random sample): 1 = the global-memory kernel instead of the shared-memory cluster kernel
 *   family 2 (attention):     1 = the multiply-add kernels instead of the tensor-core kernels,
 *                             2 = the row-tile mma.sync kernels also where the tcgen05 paths (several new tokens) apply,
 *                             3 / 4 (read when a descriptor is created) = for several new tokens the three-launch
 *                             form (scores, softmax, values) / the one-kernel form wherever it applies
 *   family 3 (matmul):        1 = the CUDA-core kernel instead of the tcgen05 kernels, 2 (read when a descriptor is
 *                             created) = the single-CTA tcgen05 kernel also where CTA pairs (cta_group::2) apply
 *   family 4 (long rows of RMSNorm / causal softmax): 1 = the register-resident kernels only, 2 = the shared-memory
 *                             ring for every row of 4096 elements and more
 * Returns STATUS_BAD_PARAM for an unknown family or a negative variant.
 */
INFINIOP_API infiniopStatus_t infiniopExtSelectKernel(int family, int variant);

/*
 * Bounded waits (no counterpart in the reference).  The kernels that wait on
 * hardware barriers for asynchronous copies (the RoPE bulk-copy pipeline, the
 * tensor-core matmul and attention kernels, the long-row ring) or on another
 * GPU's flag (the peer-memory exchange) give every wait a limit; a wait that runs out makes its
 * thread group stop, let its copies in flight land, and leave.  The call has
 * then already returned STATUS_SUCCESS, and its output is incomplete.
 * infiniopExtDeviceTimeouts reports how many groups gave up on this handle's
 * device since the library was loaded (it synchronises the device): 0 means
 * every result so far is complete.  infiniopExtSetWaitLimit sets the number of
 * polls a RoPE pipeline wait may take (0 restores the default of 2^22); it
 * exists so that a test can make the limit run out.
 */
INFINIOP_API infiniopStatus_t infiniopExtDeviceTimeouts(infiniopHandle_t handle, uint64_t *count);
INFINIOP_API infiniopStatus_t infiniopExtSetWaitLimit(infiniopHandle_t handle, uint32_t polls);

/*
 * Batched random sample: `rows` independent rows of fp16 logits
 * [rows, voc] (voc taken from the descriptor, `row_stride` elements between
 * rows) sampled in ONE launch, row r with the uniform draw random_vals[r]
 * (device array of fp32).  results is a device array of `rows` u64 indices.
 * Per-row semantics are exactly those of infiniopRandomSample
 * (reference include/ops/random_sample/random_sample.h:17-26 applied row by
 * row); the reference itself has no batched form and needs one call, one
 * workspace and four launches per row.
 */
INFINIOP_API infiniopStatus_t infiniopGetRandomSampleBatchWorkspaceSize(infiniopRandomSampleDescriptor_t desc,
                                                                        uint64_t rows, uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopRandomSampleBatch(infiniopRandomSampleDescriptor_t desc, void *workspace,
                                                        uint64_t workspace_size, void *results, void const *logits,
                                                        int64_t row_stride, uint64_t rows, void const *random_vals,
                                                        float topp, int topk, float temperature, void *stream);

/*
 * Same as infiniopRandomSampleBatch, additionally writing a per-row trace to
 * `trace` (device, 145 fp32 per row): [0] the fp32 softmax denominator,
 * [1..64] the selected top-k indices (as bit patterns), [65..128] their
 * truncated probabilities, [129..134] SM cycle counts at the kernel's phase
 * boundaries, [141..143] (shared-memory kernel) blocks replayed on integers, elements settled by the exact path,
 * blocks replayed in all, [144] the number of passes the denominator took.  Used by the parity tests to compare intermediate
 * values with the CPU oracle, not only the final index.
 */
INFINIOP_API infiniopStatus_t infiniopRandomSampleBatchTrace(infiniopRandomSampleDescriptor_t desc, void *workspace,
                                                             uint64_t workspace_size, void *results,
                                                             void const *logits, int64_t row_stride, uint64_t rows,
                                                             void const *random_vals, float topp, int topk,
                                                             float temperature, void *trace, void *stream);

/*
 * Vocabulary-sharded sampling (no counterpart in the reference, which has no
 * multi-device code).  Each rank holds columns [shard_offset, shard_offset +
 * voc_local) of the [rows, voc_total] logits; voc_local is the descriptor's voc.
 *
 *   1. infiniopRandomSampleShardLocal on every rank writes `rows` records of
 *      infiniopRandomSampleShardRecordBytes() bytes each (local maximum, local
 *      softmax sum, and in index order the candidates that can reach the global
 *      top-k).
 *   2. The host all-gathers the record buffers (rank-major: [ranks][rows][record]).
 *   3. infiniopRandomSampleShardFinish on any rank merges them: the top-k set,
 *      its tie order and the numerators are those of infiniopRandomSample on the
 *      concatenated row; the denominator is the correctly rounded sum, whereas
 *      the unsharded path reproduces the reference's sequential fp32 sum, so
 *      about one row in a thousand can pick a neighbouring candidate.
 *      *status_flag (device int, zeroed by the caller) becomes 1 when a shard
 *      had more than 128 tied candidates and the row was not sampled.
 * Only the sampling branch (topp > 0, 2 <= topk <= 64) is provided.
 */
INFINIOP_API uint64_t infiniopRandomSampleShardRecordBytes(void);
INFINIOP_API infiniopStatus_t infiniopRandomSampleShardLocal(infiniopRandomSampleDescriptor_t desc, void *records,
                                                             void const *logits, int64_t row_stride, uint64_t rows,
                                                             uint64_t shard_offset, int topk, float temperature,
                                                             void *stream);
INFINIOP_API infiniopStatus_t infiniopRandomSampleShardFinish(infiniopHandle_t handle, void *results,
                                                              void const *gathered_records, int ranks, uint64_t rows,
                                                              uint64_t voc_total, void const *random_vals, float topp,
                                                              int topk, float temperature, void *status_flag,
                                                              void *stream);

/*
 * No counterpart in the reference library.
 *
 * infiniopRandomSampleBatch for callers that cannot hand over a workspace:
 * hosts that gave all device memory to their own arena and may not call
 * cudaMalloc where they sample, or plug-ins that only ever receive input and
 * output pointers.  The per-row working copies live in a 32 MiB array that is
 * part of the library image on every GPU that loads it, so the call performs
 * no allocation of any kind (no cudaMalloc / cudaFree, no allocating library
 * routine).  Inputs, outputs and semantics are those of
 * infiniopRandomSampleBatch.
 *
 * Limits and rules:
 *  - The array is used by the kernel that serves rows of more than 262144
 *    logits (shorter rows are sampled out of shared memory and need no scratch
 *    at all, whatever their number).  For those long rows
 *    rows * round_up(voc, 256) * 2 + 256 bytes must fit in 32 MiB (40 rows of
 *    300000 logits do); larger requests return STATUS_INSUFFICIENT_WORKSPACE
 *    and print the sizes.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress with that device current); make that first call
 *    before starting any stream capture.
 *  - All calls on a device share the one array.  Each call rewrites every byte
 *    it later reads, so nothing has to be cleared between calls, but two calls
 *    that overlap on the GPU (different streams) race: serialise them.
 */
INFINIOP_API infiniopStatus_t infiniopRandomSampleBatchStatic(infiniopRandomSampleDescriptor_t desc, void *results,
                                                              void const *logits, int64_t row_stride, uint64_t rows,
                                                              void const *random_vals, float topp, int topk,
                                                              float temperature, void *stream);

/*
 * Rows of a column-sharded matrix over peer memory (no counterpart in the
 * reference, which has no multi-device code).  For vocabulary-sharded
 * sampling on the GPUs of one node: every rank holds columns
 * [col0_r, col0_r + cols_r) of a [rows, voc] fp16 matrix in a block of device
 * memory that the other ranks have opened through CUDA IPC, and needs the
 * whole rows [row0, row0 + nrows).
 *
 * infiniopExtPeerAlloc is the one call of this library that allocates device
 * memory: `bytes` of zeroed memory from cudaMalloc (so that the block can be
 * exported) and the 64-byte IPC handle to send to the other ranks' processes;
 * infiniopExtPeerOpen maps another rank's block (not the caller's own: use
 * the pointer from PeerAlloc), infiniopExtPeerClose / infiniopExtPeerFree undo
 * them.  The first 256 bytes of every block belong to the library (flags and a
 * call counter, zero at the start and never written by the caller).
 *
 * infiniopExtPeerGatherRows: `shards[r]`, `shard_row_strides[r]` (elements),
 * `shard_col0[r]`, `shard_cols[r]` describe rank r's columns as this process
 * addresses them, `flags[r]` is the start of rank r's block.  The kernel tells
 * every peer that this rank's shard is final (everything issued earlier on
 * `stream` has completed), waits for each peer's word and copies the peers'
 * columns of this rank's rows into `full` ([nrows, voc], `full_row_stride`
 * elements).  infiniopExtPeerPublishResults writes `picked` (u64[nrows], this
 * rank's results) to rows [row0, row0 + nrows) of every `results[r]` (u64
 * arrays inside the blocks), and returns to the stream only when every rank has
 * done the same: afterwards results[rank] holds all rows, and the shard may
 * be overwritten.  Every rank must issue the same sequence of these two calls.
 * Plain peer loads and stores; no multicast.  Waits are bounded (about a
 * second) and reported by infiniopExtDeviceTimeouts.  world <= 16.
 */
INFINIOP_API infiniopStatus_t infiniopExtPeerAlloc(infiniopHandle_t handle, uint64_t bytes, void **ptr,
                                                   unsigned char *ipc_handle64);
INFINIOP_API infiniopStatus_t infiniopExtPeerOpen(infiniopHandle_t handle, const unsigned char *ipc_handle64, void **ptr);
INFINIOP_API infiniopStatus_t infiniopExtPeerClose(infiniopHandle_t handle, void *ptr);
INFINIOP_API infiniopStatus_t infiniopExtPeerFree(infiniopHandle_t handle, void *ptr);
INFINIOP_API infiniopStatus_t infiniopExtPeerGatherRows(infiniopHandle_t handle, void *full, int64_t full_row_stride,
                                                        void *const *shards, const int64_t *shard_row_strides,
                                                        const uint64_t *shard_col0, const uint64_t *shard_cols,
                                                        void *const *flags, uint32_t world, uint32_t rank,
                                                        uint64_t row0, uint64_t nrows, void *stream);
INFINIOP_API infiniopStatus_t infiniopExtPeerPublishResults(infiniopHandle_t handle, void *const *results,
                                                            const void *picked, void *const *flags, uint32_t world,
                                                            uint32_t rank, uint64_t row0, uint64_t nrows, void *stream);

/*
 * The same exchange folded into the sampling kernel: ONE launch waits for the
 * peers' shards, samples rows [row0, row0 + nrows) out of them with peer
 * loads, stores every index into every rank's result array and closes with
 * the "done" round.  `desc` describes whole rows (voc = world * shard_cols).
 * Conditions: topp > 0, 2 <= topk <= 64, voc <= 262144, equal shards of a
 * multiple of 8 columns, nrows >= 1; otherwise STATUS_BAD_PARAM, and the three
 * calls above (GatherRows, infiniopRandomSampleBatch, PublishResults) apply.
 * A rank without rows takes part with GatherRows and PublishResults (nrows 0).
 */
INFINIOP_API infiniopStatus_t infiniopRandomSampleBatchPeer(infiniopRandomSampleDescriptor_t desc, void *const *results,
                                                            void *const *shards, const int64_t *shard_row_strides,
                                                            uint64_t shard_cols, void *const *flags, uint32_t world,
                                                            uint32_t rank, uint64_t row0, uint64_t nrows,
                                                            void const *random_vals, float topp, int topk,
                                                            float temperature, void *stream);

#endif /* INFINIOP_B200_EXT_H */
