/*
 * infiniop_ext.h - additive entry points of the B200 backend that have no
 * counterpart in the reference library.  Nothing here changes the behaviour of
 * the reference-shaped ABI in infiniop.h.
 */
#ifndef INFINIOP_B200_EXT_H
#define INFINIOP_B200_EXT_H

#include "infiniop.h"

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
 * truncated probabilities, [129..143] SM cycle counts at the kernel's phase
 * boundaries, [144] the number of passes the denominator took.  Used by the parity tests to compare intermediate
 * values with the CPU oracle, not only the final index.
 */
INFINIOP_API infiniopStatus_t infiniopRandomSampleBatchTrace(infiniopRandomSampleDescriptor_t desc, void *workspace,
                                                             uint64_t workspace_size, void *results,
                                                             void const *logits, int64_t row_stride, uint64_t rows,
                                                             void const *random_vals, float topp, int topk,
                                                             float temperature, void *trace, void *stream);

#endif /* INFINIOP_B200_EXT_H */
