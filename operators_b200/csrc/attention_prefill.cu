// Attention with several new tokens per call (prefill, speculative decoding) on the tensor cores.
//
// The reference composite (src/ops/attention/operator.cc:252-305) runs, after the two rearranges into the caches:
// a cuBLAS matmul q k^T scaled by 1/sqrt(dh) into an fp16 score tensor, the causal softmax in place, a second
// matmul with v, and a rearrange of the result to [seq, n_q_head, dh].  This path keeps that structure and its
// two fp16 roundings (the score after the scaling, the probability after the division by the whole row's sum),
// with this library's own kernels:
//   1. scores[h] = alpha * q[h] k_cache[h / group]^T     tcgen05 matmul (tc_gemm.cuh), one batch entry per q head,
//                                                         K read as a K-major operand straight from the cache
//   2. causal softmax in place on scores                  causal_softmax.cu (masked tails never read)
//   3. out[:, h, :] = scores[h] v_cache[h / group]        tcgen05 matmul, V read as an MN-major operand from the
//                                                         cache, the result rows written with out's strides, so
//                                                         the closing rearrange is part of the epilogue
// K and V are read once per q head from L2 instead of once per 8 query rows, and the products run on TMEM
// accumulators.  One new token per call keeps the dedicated decode kernels of attention.cu.
#include "attention_prefill.cuh"

#include <new>

namespace b200 {

struct AttnPrefill {
    int device_id;
    uint32_t nh, seq, total, total_pad;
    MatmulPlan scores, values;
    TcMapCache scores_maps, values_maps;
    infiniopCausalSoftmaxDescriptor_t softmax;
    uint64_t scores_bytes, scratch_bytes;
};

AttnPrefill *attn_prefill_create(infiniopHandle_t handle, const AttnPrefillShape &s, uint64_t *workspace_bytes) {
    auto *h = reinterpret_cast<Handle *>(handle);
    if (s.dh % 8 != 0 || s.seq == 0 || s.total == 0) return nullptr;
    auto *p = new (std::nothrow) AttnPrefill{};
    if (p == nullptr) return nullptr;
    p->device_id = h->device_id;
    p->nh = s.nh, p->seq = s.seq, p->total = s.total;
    p->total_pad = (s.total + 7) / 8 * 8;// rows of the score tensor stay 16-byte aligned
    p->softmax = nullptr;
    p->scores.counter_slot = p->values.counter_slot = -1;

    const uint32_t nkvh = s.nh / s.group;
    uint64_t sc_shape[3] = {s.nh, s.seq, s.total};
    int64_t sc_strides[3] = {(int64_t) s.seq * p->total_pad, (int64_t) p->total_pad, 1};
    TensorDescriptor sc{F16, 3, sc_shape, sc_strides};
    uint64_t q_shape[3] = {s.nh, s.seq, s.dh};
    int64_t q_strides[3] = {s.q_s0, s.q_s1, 1};
    TensorDescriptor qd{F16, 3, q_shape, q_strides};
    uint64_t kt_shape[3] = {nkvh, s.dh, s.total};// k_cache[kv head]^T: [dh, total]
    int64_t kt_strides[3] = {s.kc_s0, 1, s.kc_s1};
    TensorDescriptor kt{F16, 3, kt_shape, kt_strides};
    uint64_t v_shape[3] = {nkvh, s.total, s.dh};
    int64_t v_strides[3] = {s.vc_s0, s.vc_s1, 1};
    TensorDescriptor vd{F16, 3, v_shape, v_strides};
    uint64_t o_shape[3] = {s.nh, s.seq, s.dh};// out[seq, nh, dh] seen per head
    int64_t o_strides[3] = {(int64_t) s.dh, (int64_t) s.nh * s.dh, 1};
    TensorDescriptor od{F16, 3, o_shape, o_strides};

    const float alpha = (float) (1.0 / sqrt((double) s.dh));// `float qk_alpha = 1 / sqrt(head_dim)`, operator.cc:136
    bool ok = matmul_plan_create(p->scores, h, &sc, alpha, &qd, &kt, 0.f, tc::kEpiPlain, s.group) == STATUS_SUCCESS &&
              p->scores.use_tc;
    ok = ok && matmul_plan_create(p->values, h, &od, 1.f, &sc, &vd, 0.f, tc::kEpiPlain, s.group) == STATUS_SUCCESS &&
         p->values.use_tc;
    ok = ok && infiniopCreateCausalSoftmaxDescriptor(handle, &p->softmax, &sc) == STATUS_SUCCESS;
    if (ok) {
        // causal structure: score tiles wholly behind the mask are never read by the softmax (it writes their zeros
        // itself), and a row block's probabilities are zero beyond its last row's mask
        for (MatmulPlan *pl : {&p->scores, &p->values}) {
            if (!pl->swapped && !pl->g.streamk) {
                pl->g.causal_mode = pl == &p->scores ? 1u : 2u;
                pl->g.causal_seq = s.seq, pl->g.causal_total = s.total;
            }
        }
    }
    if (!ok) {
        attn_prefill_destroy(p);
        return nullptr;
    }
    auto pad = [](uint64_t b) { return (b + 255) / 256 * 256; };
    p->scores_bytes = pad((uint64_t) s.nh * s.seq * p->total_pad * 2);
    p->scratch_bytes = pad(p->scores.workspace_bytes > p->values.workspace_bytes ? p->scores.workspace_bytes
                                                                                 : p->values.workspace_bytes);
    *workspace_bytes = p->scores_bytes + p->scratch_bytes + 256;
    return p;
}

infiniopStatus_t attn_prefill_run(AttnPrefill *p, void *workspace, void *out, const void *q, const void *k_cache,
                                  const void *v_cache, cudaStream_t st) {
    auto *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t) 255);
    void *scores = base, *scratch = base + p->scores_bytes;
    infiniopStatus_t s = matmul_plan_run(p->scores, p->scores_maps, scratch, p->scratch_bytes, scores, q, k_cache, st);
    if (s != STATUS_SUCCESS) return s;
    s = infiniopCausalSoftmax(p->softmax, nullptr, 0, scores, st);
    if (s != STATUS_SUCCESS) return s;
    return matmul_plan_run(p->values, p->values_maps, scratch, p->scratch_bytes, out, scores, v_cache, st);
}

void attn_prefill_destroy(AttnPrefill *p) {
    if (p == nullptr) return;
    if (p->softmax != nullptr) infiniopDestroyCausalSoftmaxDescriptor(p->softmax);
    matmul_plan_destroy(p->scores);
    matmul_plan_destroy(p->values);
    delete p;
}

}// namespace b200
