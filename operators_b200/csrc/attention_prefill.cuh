// Interface between the attention entry points (attention.cu) and the tensor-core path for calls with several
// new tokens (attention_prefill.cu).
#pragma once
#include "matmul.cuh"

namespace b200 {

struct AttnPrefillShape {
    uint32_t nh, group, seq, dh, total;
    int64_t q_s0, q_s1, kc_s0, kc_s1, vc_s0, vc_s1;// element strides of q [nh, seq, dh] and the caches [nkvh, buf, dh]
};

struct AttnPrefill;
// nullptr when the layouts cannot go through TMA descriptors (the caller keeps its other kernels).
AttnPrefill *attn_prefill_create(infiniopHandle_t handle, const AttnPrefillShape &shape, uint64_t *workspace_bytes);
// After the new k and v rows are in the caches.  `workspace` holds *workspace_bytes of attn_prefill_create.
infiniopStatus_t attn_prefill_run(AttnPrefill *p, void *workspace, void *out, const void *q, const void *k_cache,
                                  const void *v_cache, cudaStream_t stream);
void attn_prefill_destroy(AttnPrefill *p);

// The same computation in one kernel (attention_fused.cu): head sizes that are multiples of 8 up to 256, no workspace.  nullptr when the
// shape or the strides do not fit it.
struct AttnFused;
AttnFused *attn_fused_create(infiniopHandle_t handle, const AttnPrefillShape &shape);
infiniopStatus_t attn_fused_run(AttnFused *f, void *out, const void *q, const void *k_cache, const void *v_cache,
                                cudaStream_t stream);
void attn_fused_destroy(AttnFused *f);
// CTAs (one cluster) that share a block of 128 query rows of this shape, each with a range of the cached tokens.
uint32_t attn_fused_splits(const AttnPrefillShape &shape, int sm_count, int device_id);
// Waits that ran out of time inside the fused kernel since the library was loaded (synchronises); ~0 on error.
unsigned long long attn_fused_timeouts_read();

}// namespace b200
