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

// Rows whose columns are split over `world` ranks' memories (vocabulary-sharded logits on the GPUs of one node,
// blocks opened through CUDA IPC; peer_exchange.cu describes the flag words).  world == 0: `logits` holds whole rows.
constexpr uint32_t kPeerMaxRanks = 16;
constexpr uint32_t kPeerReady = 0, kPeerDone = 16, kPeerCalls = 32, kPeerFinished = 33;// 32-bit words of a flag block
struct PeerRowSource {
    uint32_t world, rank;
    uint32_t shard_vecs;                 // 128-bit vectors per shard row: equal shards of a multiple of 8 columns
    uint32_t rows;                       // rows of this launch (= leader CTAs that report back)
    uint64_t row0;                       // this rank's first row within the shards and the result arrays
    const uint16_t *shard[kPeerMaxRanks];// rank r's [all rows, shard_vecs * 8] logits as this process addresses them
    int64_t shard_stride[kPeerMaxRanks]; // elements between its rows
    uint32_t *flags[kPeerMaxRanks];      // rank r's flag words
    unsigned long long *results[kPeerMaxRanks];// rank r's result array (all rows)
};

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
    // Sharded rows (pair kernel only): the row is read from the peers' shards after their "shard is final" words have
    // arrived, the index goes to every rank's result array, and the launch ends with the "done" round of the protocol.
    PeerRowSource peer;
};

// Shared-memory resident cluster form (random_sample_pair.cu): sampling branch, voc <= 262144.
bool random_sample_pair_supported(int voc);
infiniopStatus_t random_sample_pair_launch(const RandomSampleArgs &args, int rows, cudaStream_t stream);
// Waits on a peer's flag word that ran out inside the pair kernel since the library was loaded (synchronises).
unsigned long long random_sample_pair_timeouts_read();

bool random_sample_uses_workspace(const RandomSampleArgs &args);
uint64_t random_sample_work_pitch(int voc);
uint64_t random_sample_workspace_bytes(int voc, int rows);
infiniopStatus_t random_sample_launch(const RandomSampleArgs &args, int rows, void *workspace, uint64_t workspace_size,
                                      cudaStream_t stream);

}// namespace b200
