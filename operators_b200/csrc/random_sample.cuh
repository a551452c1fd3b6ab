// Launch interface of the random-sample kernel, shared by the reference-shaped
// single-row entry point and the batched extension.
#pragma once
#include "common.cuh"

namespace b200 {

// Object behind infiniopRandomSampleDescriptor_t.
struct RandomSampleDesc {
    Device device;
    int device_id;
    int sm_count;
    int voc;
    int result_len;
};

constexpr int kDebugStride = 1 + 2 * 64 + 16;// floats per row of the optional trace buffer

struct RandomSampleArgs {
    const uint16_t *logits; // fp16 rows
    int64_t logits_stride;  // elements between rows
    uint16_t *work;         // per-row working copy of the row as 16-bit keys
    int64_t work_pitch;     // elements between working rows (multiple of 256)
    uint64_t *result;       // one index per row
    int64_t result_stride;
    const float *random_vals;// device array of per-row uniform draws, or NULL to use random_val
    float random_val;
    float topp;
    int topk;
    float temperature;
    int voc;
    // Optional device trace per row: [0] = softmax denominator S, [1..64] = the
    // top-k indices (bit patterns), [65..128] = their truncated probabilities,
    // [129..144] = SM cycle counts at the phase boundaries (relative to entry)
    // followed by the number of denominator passes.
    float *debug;
};

// Shared-memory resident cluster form (random_sample_pair.cu): sampling branch, voc <= 262144.
bool random_sample_pair_supported(int voc);
infiniopStatus_t random_sample_pair_launch(const RandomSampleArgs &args, int rows, cudaStream_t stream);

bool random_sample_uses_workspace(const RandomSampleArgs &args);
uint64_t random_sample_work_pitch(int voc);
uint64_t random_sample_workspace_bytes(int voc, int rows);
infiniopStatus_t random_sample_launch(const RandomSampleArgs &args, int rows, void *workspace, uint64_t workspace_size,
                                      cudaStream_t stream);

}// namespace b200
