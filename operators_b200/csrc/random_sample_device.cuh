// Device-side pieces shared by the sampling kernels: 16-bit order-preserving
// keys, the exponential term and the sorted top-k buffer with the reference's
// insertion cascade.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kSlots = 64;// top-k buffer slots held by one warp (2 per lane)

// ---- 16-bit order-preserving keys -------------------------------------------
// key in [1, 65535]; +0 and -0 share 0x8000 (they compare equal as floats);
// 0 is reserved for "no element" (padding of the working copy).
__device__ __forceinline__ uint32_t key_of(uint16_t h) {
    const uint32_t mag = h & 0x7FFFu;
    return (h & 0x8000u) ? (0x8000u - mag) : (0x8000u + mag);
}
__device__ __forceinline__ float val_of(uint32_t key) {
    const uint16_t h = key >= 0x8000u ? (uint16_t) (key - 0x8000u) : (uint16_t) (0x8000u | (0x8000u - key));
    return f16_to_f32(h);
}

// expf((v - M) / T) as the reference forms it: fp32 subtract, IEEE fp32 divide,
// then the exponential, here correctly rounded through double.
__device__ __forceinline__ float term_of(float v, float M, float T) {
    const float x = __fdiv_rn(__fsub_rn(v, M), T);
    return __double2float_rn(exp((double) x));
}

// ---- sorted top-k buffer of warp 0: slot s lives in lane s % 32, register s / 32
struct TopBuf {
    uint32_t k0, k1;// keys (0 = empty)
    uint32_t i0, i1;// indices
};

// Streaming insertion of (ck, ci) with the reference's strict-greater cascade.
// Slots holding keys >= ck form a prefix of length s1; the new element lands in
// slot s1; every later slot that starts a run of equal keys receives the first
// element of the run before it (for distinct keys this is a plain shift by one);
// what leaves slot k-1 is dropped.
__device__ __forceinline__ void topbuf_insert(TopBuf &b, int lane, int k, uint32_t ck, uint32_t ci) {
    const uint32_t ge0 = __ballot_sync(0xffffffffu, b.k0 >= ck);
    const uint32_t ge1 = __ballot_sync(0xffffffffu, b.k1 >= ck);
    const int s1 = __popc(ge0) + __popc(ge1);
    if (s1 >= k) return;
    // key of the slot to the left
    uint32_t left0 = __shfl_up_sync(0xffffffffu, b.k0, 1);
    uint32_t left1 = __shfl_up_sync(0xffffffffu, b.k1, 1);
    const uint32_t k0_last = __shfl_sync(0xffffffffu, b.k0, 31);
    if (lane == 0) {
        left0 = 0xFFFFFFFFu;
        left1 = k0_last;
    }
    const bool rs0 = b.k0 != left0, rs1 = b.k1 != left1;// slot starts a run
    const unsigned long long RS = (unsigned long long) __ballot_sync(0xffffffffu, rs0) |
                                  ((unsigned long long) __ballot_sync(0xffffffffu, rs1) << 32) | (1ull << s1);
    const int p0 = lane, p1 = lane + 32;
    // start of the previous run for a run-start slot p > s1
    int q0 = 0, q1 = 0;
    const bool mv0 = p0 > s1 && rs0, mv1 = p1 > s1 && rs1;
    if (mv0) q0 = 63 - __clzll(RS & ((1ull << p0) - 1ull));
    if (mv1) q1 = 63 - __clzll(RS & ((1ull << p1) - 1ull));
    // fetch old index at slot q (both registers of the source lane)
    const uint32_t f0a = __shfl_sync(0xffffffffu, b.i0, q0 & 31), f0b = __shfl_sync(0xffffffffu, b.i1, q0 & 31);
    const uint32_t f1a = __shfl_sync(0xffffffffu, b.i0, q1 & 31), f1b = __shfl_sync(0xffffffffu, b.i1, q1 & 31);
    if (mv0) {
        b.k0 = left0;
        b.i0 = q0 < 32 ? f0a : f0b;
    }
    if (mv1) {
        b.k1 = left1;
        b.i1 = q1 < 32 ? f1a : f1b;
    }
    if (p0 == s1) {
        b.k0 = ck;
        b.i0 = ci;
    }
    if (p1 == s1) {
        b.k1 = ck;
        b.i1 = ci;
    }
    if (p0 >= k) b.k0 = 0;
    if (p1 >= k) b.k1 = 0;
}

// Top-p cut and pick over the k truncated probabilities p[0..k) of the top-k, in
// the reference's order of operations (reference
// src/ops/random_sample/cpu/random_sample.cc:99-128).  One thread calls it.
// Nothing is written when no prefix sum exceeds the scaled draw, as in the
// reference.
__device__ __forceinline__ void pick_from_topk(const float *p, const uint32_t *idx, int k, float topp,
                                               float random_val, uint64_t *out) {
    float acc = 0.f;
    int end = 0;
    for (end = 0; end < k; ++end) {
        acc = __fadd_rn(acc, p[end]);
        if (acc >= topp) break;
    }
    end = end < k - 1 ? end + 1 : k;
    float sum_s = 0.f;
    for (int i = 0; i < end; ++i) sum_s = __fadd_rn(sum_s, p[i]);
    const float r = __fmul_rn(random_val, sum_s);
    sum_s = 0.f;
    for (int i = 0; i < end; ++i) {
        sum_s = __fadd_rn(sum_s, p[i]);
        if (r < sum_s) {
            *out = idx[i];
            return;
        }
    }
}

}// namespace b200
