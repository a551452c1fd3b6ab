// Random sample: temperature / top-k / top-p sampling (or argmax) over rows of
// fp16 logits, reproducing the reference CPU backend's result index exactly.
//
// Replaces reference src/ops/random_sample/cuda/random_sample.cu:7-180 and
// src/ops/random_sample/cuda/random_sample_cuda.cc:5-37 behind
// include/ops/random_sample/random_sample.h.  The behaviour that is matched is
// the CPU backend's (src/ops/random_sample/cpu/random_sample.cc:45-185), which
// differs from the reference's own nv-gpu pipeline (that one normalises over
// the top-k only).  What the CPU code does, restated as what has to be computed:
//
//  (1) k passes of swap selection leave the k largest values in slots 0..k-1,
//      descending.  Re-ordering the compare-exchanges column by column shows
//      this is a STREAMING INSERTION of the elements, in index order, into a
//      sorted buffer of k slots where an element moves past a slot only when it
//      is strictly greater; the element that falls off the end stays at the
//      position of the element that was streamed in.  Hence
//        - the tie order inside the top-k is that of the insertion cascade, and
//        - position j >= k ends up holding min(a_j, tau_{j-1}), tau_{j-1} being
//          the k-th largest value among a_0..a_{j-1}.
//  (2) S = sum over that permuted row of expf((v - M) / T), accumulated
//      sequentially in fp32.  Within one binade of the running sum every
//      addition changes it by an integer number of ulps, round-to-nearest-even
//      of term/ulp, so the tail of the sum is an integer sum that can be formed
//      in any order; only exact half-way cases and the additions that carry
//      the sum into the next binade are order dependent.  Those are located per
//      256-element block and replayed serially with real fp32 additions.
//  (3) p_i = trunc16(expf((v_i - M) / T) / S) for the top-k, the top-p cut and
//      the pick with the caller's uniform draw, all in the reference's order.
//
// expf: the host libm's expf is within 0.502 ulp; here every term comes from a
// double-precision exp rounded once to fp32 (correct rounding).  The two differ
// by one fp32 ulp for about 8e-5 of all arguments, far below what can move a
// truncated fp16 probability.
//
// One CTA of 1024 threads owns a row.  The row is converted once to 16-bit
// order-preserving keys in the caller's workspace (L2 resident afterwards);
// positions that step (1) overwrites are patched in that copy.
#include "common.cuh"
#include "random_sample.cuh"
#include "random_sample_device.cuh"

#include <cooperative_groups.h>

#include <cstdlib>
#include <atomic>
#include <new>

using namespace b200;

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kBlk = 256;     // elements per block: one 128-bit vector per lane of a warp
constexpr int kListCap = 64;  // ordered per-warp list capacity (candidates / flagged records)
constexpr uint32_t kEmptyMin = 0xFFFFFFFFu;


struct Shared {
    uint32_t list_idx[kWarps][kListCap];
    uint16_t list_key[kWarps][kListCap];
    int list_cnt[kWarps];
    int overflow;
    uint32_t top_key[kSlots];
    uint32_t top_idx[kSlots];
    float top_term[kSlots];
    float blk_terms[kBlk];
    uint32_t red_u32[kWarps];
    unsigned long long red_u64[kWarps];
    float s;           // running fp32 sum
    uint32_t pos;      // first position of the row not yet folded into s
    int done;
};

// Append the flagged elements of one 256-element block (8 per lane, `mask` has
// bit e set for element e of this lane) to this warp's list, in index order.
__device__ __forceinline__ void warp_append(Shared &sm, int warp, int lane, uint32_t mask, const uint32_t keys[8],
                                            uint32_t base_idx) {
    const uint32_t any = __ballot_sync(0xffffffffu, mask != 0);
    if (any == 0) return;
    const int cnt = __popc(mask);
    int pre = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, pre, o);
        if (lane >= o) pre += n;
    }
    const int total = __shfl_sync(0xffffffffu, pre, 31);
    const int start = sm.list_cnt[warp];
    int at = start + pre - cnt;
    if (start + total > kListCap) {
        if (lane == 0) sm.overflow = 1;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (mask & (1u << e)) {
                sm.list_idx[warp][at] = base_idx + lane * 8 + e;
                sm.list_key[warp][at] = (uint16_t) keys[e];
                ++at;
            }
        }
    }
    __syncwarp();
    if (lane == 0) sm.list_cnt[warp] = start + total > kListCap ? kListCap + 1 : start + total;
    __syncwarp();
}

__device__ __forceinline__ void load_keys(const uint16_t *work, uint32_t base, int lane, uint32_t keys[8]) {
    const uint4 v = *reinterpret_cast<const uint4 *>(work + base + lane * 8);
    const uint32_t *p = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        keys[2 * k] = p[k] & 0xFFFFu;
        keys[2 * k + 1] = p[k] >> 16;
    }
}

// ---- running multiset of the k largest values seen so far (values only) -----
struct MinBuf {
    uint32_t v0, v1;// kEmptyMin in slots >= k
    uint32_t tau;   // smallest held value == k-th largest so far
};
__device__ __forceinline__ void minbuf_replace(MinBuf &m, int lane, uint32_t key) {
    const uint32_t h0 = __ballot_sync(0xffffffffu, m.v0 == m.tau);
    if (h0) {
        if (lane == __ffs(h0) - 1) m.v0 = key;
    } else {
        const uint32_t h1 = __ballot_sync(0xffffffffu, m.v1 == m.tau);
        if (lane == __ffs(h1) - 1) m.v1 = key;
    }
    m.tau = __reduce_min_sync(0xffffffffu, min(m.v0, m.v1));
}

// Warp 0 walks one 256-element block and feeds every element that beats the
// running k-th largest value, in index order.  Elements below `first` are
// skipped.  A record at position j is replaced by tau_{j-1} in the working copy.
__device__ __forceinline__ void records_direct_block(uint16_t *work, uint32_t blk_base, uint32_t first, int lane,
                                                     MinBuf &m) {
    uint32_t keys[8];
    load_keys(work, blk_base, lane, keys);
    uint32_t mask = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const uint32_t j = blk_base + lane * 8 + e;
        if (j >= first && keys[e] > m.tau) mask |= 1u << e;
    }
    uint32_t any = __ballot_sync(0xffffffffu, mask != 0);
    while (any) {
        const int src = __ffs(any) - 1;
        const uint32_t smask = __shfl_sync(0xffffffffu, mask, src);
        const int e = __ffs(smask) - 1;
        uint32_t key = 0;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            if (t == e) key = keys[t];
        }
        key = __shfl_sync(0xffffffffu, key, src);
        if (key > m.tau) {
            if (lane == 0) work[blk_base + src * 8 + e] = (uint16_t) m.tau;
            minbuf_replace(m, lane, key);
        }
        if (lane == src) mask &= mask - 1;
        any = __ballot_sync(0xffffffffu, mask != 0);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
    random_sample_kernel(RandomSampleArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Shared &sm = *reinterpret_cast<Shared *>(smem_raw);
    uint32_t *blk_sum = reinterpret_cast<uint32_t *>(smem_raw + sizeof(Shared));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x;
    const int n = a.voc;
    const uint16_t *logits = a.logits + (int64_t) row * a.logits_stride;
    uint16_t *work = a.work + (int64_t) row * a.work_pitch;
    const float random_val = a.random_vals ? a.random_vals[row] : a.random_val;
    const uint32_t nblk = (uint32_t) ((n + kBlk - 1) / kBlk);
    const uint32_t npad = nblk * kBlk;

    const bool sampling = a.topp > 0.f && a.topk > 1;
    int k = a.topk > n ? n : a.topk;
    const long long t_entry = clock64();
    int stamp_i = 0;
    auto stamp = [&]() {// phase boundary -> trace buffer (thread 0, only when tracing)
        if (a.debug && tid == 0 && stamp_i < 15) {
            a.debug[(int64_t) row * kDebugStride + 129 + stamp_i] = (float) (clock64() - t_entry);
        }
        ++stamp_i;
    };

    // ---- pass A: logits -> keys (working copy), per-thread and row maximum --
    const bool in_aligned = (reinterpret_cast<uintptr_t>(logits) & 15u) == 0;
    uint32_t tmax = 0;
    unsigned long long best = 0;// argmax: (key << 32) | ~index
    constexpr int kInFlight = 4;// 128-bit loads per thread issued before any is consumed
    for (uint32_t base0 = tid * 8; base0 < npad; base0 += kThreads * 8 * kInFlight) {
        uint4 raw[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t base = base0 + u * kThreads * 8;
            if (in_aligned && base + 8 <= (uint32_t) n) raw[u] = ld_stream(logits + base);
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t base = base0 + u * kThreads * 8;
            if (base >= npad) break;
            uint32_t keys[8];
            if (in_aligned && base + 8 <= (uint32_t) n) {
                const uint32_t *p = reinterpret_cast<const uint32_t *>(&raw[u]);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    keys[2 * q] = key_of((uint16_t) (p[q] & 0xFFFFu));
                    keys[2 * q + 1] = key_of((uint16_t) (p[q] >> 16));
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) keys[e] = base + e < (uint32_t) n ? key_of(logits[base + e]) : 0u;
            }
            uint4 o;
            o.x = keys[0] | (keys[1] << 16);
            o.y = keys[2] | (keys[3] << 16);
            o.z = keys[4] | (keys[5] << 16);
            o.w = keys[6] | (keys[7] << 16);
            if (sampling) *reinterpret_cast<uint4 *>(work + base) = o;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                tmax = max(tmax, keys[e]);
                const unsigned long long cand = ((unsigned long long) keys[e] << 32) | (0xFFFFFFFFu - (base + e));
                best = cand > best ? cand : best;
            }
        }
    }

    if (!sampling) {
        // argmax, lowest index among equal maxima (reference random_sample.cc:130-153)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) sm.red_u64[warp] = best;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < kWarps; ++w) best = sm.red_u64[w] > best ? sm.red_u64[w] : best;
            a.result[(int64_t) row * a.result_stride] = 0xFFFFFFFFu - (uint32_t) (best & 0xFFFFFFFFu);
        }
        return;
    }

    stamp();// 0: row converted to keys
    if (tid < kWarps) sm.list_cnt[tid] = 0;
    if (tid == 0) {
        sm.overflow = 0;
        sm.done = 0;
    }
    // Lower bound L of the k-th largest key: the k-th largest per-thread maximum
    // (k distinct elements are >= it).  Largest L with count(tmax >= L) >= k.
    uint32_t lo = 1, hi = 65535;
    bool have_lt_k;
    {
        const int have = __syncthreads_count(tmax >= 1);
        const int need = k < have ? k : have;
        have_lt_k = have < k;
        while (lo < hi) {
            const uint32_t mid = (lo + hi + 1) >> 1;
            if (__syncthreads_count(tmax >= mid) >= need) lo = mid;
            else hi = mid - 1;
        }
    }
    // Fewer than k threads hold data (tiny rows): every element is a candidate.
    const uint32_t L = have_lt_k ? 1u : lo;
    __syncthreads();// working copy and list counters visible to the whole CTA
    stamp();// 1: lower bound of the k-th largest key

    // ---- pass B: candidates (key >= L) in index order ------------------------
    const uint32_t span = (nblk + kWarps - 1) / kWarps;// blocks per warp, contiguous
    {
        const uint32_t b_begin = warp * span, b_end = min(nblk, b_begin + span);
        for (uint32_t b = b_begin; b < b_end; ++b) {
            uint32_t keys[8];
            load_keys(work, b * kBlk, lane, keys);
            uint32_t mask = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e) mask |= (keys[e] >= L ? 1u : 0u) << e;
            warp_append(sm, warp, lane, mask, keys, b * kBlk);
        }
    }
    __syncthreads();
    stamp();// 2: candidate lists

    // ---- exact top-k with the reference's tie order (warp 0) -----------------
    TopBuf tb{0, 0, 0, 0};
    if (warp == 0) {
        if (!sm.overflow) {
            for (int w = 0; w < kWarps; ++w) {
                const int cnt = sm.list_cnt[w];
                for (int c = 0; c < cnt; ++c) topbuf_insert(tb, lane, k, sm.list_key[w][c], sm.list_idx[w][c]);
            }
        } else {
            // More ties than the lists hold: stream the whole row, skipping
            // blocks that cannot change a full buffer.
            for (uint32_t b = 0; b < nblk; ++b) {
                uint32_t keys[8];
                load_keys(work, b * kBlk, lane, keys);
                const uint32_t kth = __shfl_sync(0xffffffffu, (k - 1) < 32 ? tb.k0 : tb.k1, (k - 1) & 31);
                uint32_t mask = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) mask |= (keys[e] > kth ? 1u : 0u) << e;
                uint32_t any = __ballot_sync(0xffffffffu, mask != 0);
                while (any) {
                    const int src = __ffs(any) - 1;
                    const uint32_t smask = __shfl_sync(0xffffffffu, mask, src);
                    const int e = __ffs(smask) - 1;
                    uint32_t key = 0;
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        if (t == e) key = keys[t];
                    }
                    key = __shfl_sync(0xffffffffu, key, src);
                    topbuf_insert(tb, lane, k, key, b * kBlk + src * 8 + e);
                    if (lane == src) mask &= mask - 1;
                    any = __ballot_sync(0xffffffffu, mask != 0);
                }
            }
        }
        sm.top_key[lane] = tb.k0;
        sm.top_key[lane + 32] = tb.k1;
        sm.top_idx[lane] = tb.i0;
        sm.top_idx[lane + 32] = tb.i1;
    }
    __syncthreads();
    stamp();// 3: top-k in order
    const float M = val_of(sm.top_key[0]);
    const float T = a.temperature;

    // ---- positions j >= k: replace records by tau_{j-1} in the working copy --
    if ((uint32_t) k < (uint32_t) n) {
        MinBuf mb{kEmptyMin, kEmptyMin, 0};
        if (warp == 0) {
            if (lane < k) mb.v0 = work[lane];
            if (lane + 32 < k) mb.v1 = work[lane + 32];
            mb.tau = __reduce_min_sync(0xffffffffu, min(mb.v0, mb.v1));
        }
        // Head of the row: warp 0 alone, block by block.  Afterwards tiles that
        // double in length: the whole CTA flags elements above the tile-start
        // tau into ordered lists, warp 0 replays them.
        const uint32_t head_blocks = min(nblk, 8u);
        if (warp == 0) {
            for (uint32_t b = 0; b < head_blocks; ++b) records_direct_block(work, b * kBlk, (uint32_t) k, lane, mb);
            if (lane == 0) sm.red_u32[0] = mb.tau;
        }
        uint32_t t_begin = head_blocks;
        while (t_begin < nblk) {// uniform across the CTA
            const uint32_t t_end = min(nblk, t_begin * 2);
            if (tid < kWarps) sm.list_cnt[tid] = 0;
            if (tid == 0) sm.overflow = 0;
            __syncthreads();
            const uint32_t tau0 = sm.red_u32[0];
            const uint32_t tspan = (t_end - t_begin + kWarps - 1) / kWarps;
            const uint32_t b_begin = t_begin + warp * tspan, b_end = min(t_end, b_begin + tspan);
            for (uint32_t b = b_begin; b < b_end; ++b) {
                uint32_t keys[8];
                load_keys(work, b * kBlk, lane, keys);
                uint32_t mask = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) mask |= (keys[e] > tau0 ? 1u : 0u) << e;
                warp_append(sm, warp, lane, mask, keys, b * kBlk);
            }
            __syncthreads();
            if (warp == 0) {
                if (!sm.overflow) {
                    for (int w = 0; w < kWarps; ++w) {
                        const int cnt = sm.list_cnt[w];
                        for (int c = 0; c < cnt; ++c) {
                            const uint32_t key = sm.list_key[w][c];
                            if (key > mb.tau) {
                                if (lane == 0) work[sm.list_idx[w][c]] = (uint16_t) mb.tau;
                                minbuf_replace(mb, lane, key);
                            }
                        }
                    }
                } else {
                    for (uint32_t b = t_begin; b < t_end; ++b) records_direct_block(work, b * kBlk, (uint32_t) k, lane, mb);
                }
                if (lane == 0) sm.red_u32[0] = mb.tau;
            }
            t_begin = t_end;
            __syncthreads();
        }
    }
    __syncthreads();
    stamp();// 4: records patched

    // ---- denominator S: sequential fp32 sum over the permuted row ------------
    if (warp == 0) {
        for (int i = lane; i < k; i += 32) sm.top_term[i] = term_of(val_of(sm.top_key[i]), M, T);
        __syncwarp();
        if (lane == 0) {
            float s = 0.f;
            for (int i = 0; i < k; ++i) s = __fadd_rn(s, sm.top_term[i]);
            sm.s = s;
            sm.pos = (uint32_t) k;
            sm.done = (uint32_t) k >= (uint32_t) n;
        }
    }
    __syncthreads();

    stamp();// 5: top-k terms summed
    uint32_t pass = 0;
    for (; pass <= nblk && !sm.done; ++pass) {// a pass ends at the first order-dependent block
        const float s = sm.s;
        const uint32_t pos = sm.pos;
        const uint32_t sbits = __float_as_uint(s);
        const int e_s = (int) ((sbits >> 23) & 0xFFu);
        const uint32_t m0 = (sbits & 0x7FFFFFu) | 0x800000u;
        // terms below half an ulp of s cannot change it: v below this cut is skipped
        const float ulp_half = __uint_as_float((uint32_t) max(e_s - 24, 1) << 23);
        const float v_cut = M + T * (logf(ulp_half) - 0.01f) - 0.01f * fabsf(M) - 0.01f;
        const uint32_t b_first = pos / kBlk;
        const uint32_t bspan = (nblk - b_first + kWarps - 1) / kWarps;
        const uint32_t b_begin = b_first + warp * bspan, b_end = min(nblk, b_begin + bspan);
        for (uint32_t b = b_begin; b < b_end; ++b) {
            uint32_t keys[8];
            load_keys(work, b * kBlk, lane, keys);
            uint32_t csum = 0;
            bool tie = false;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t j = b * kBlk + lane * 8 + e;
                if (keys[e] == 0 || j < pos) continue;
                const float v = val_of(keys[e]);
                if (v < v_cut) continue;
                const uint32_t tb_ = __float_as_uint(term_of(v, M, T));
                int e_t = (int) ((tb_ >> 23) & 0xFFu);
                uint32_t man = tb_ & 0x7FFFFFu;
                if (e_t == 0) e_t = 1;
                else man |= 0x800000u;
                const int d = e_s - e_t;// >= 0: every term is <= 1 <= s
                if (d >= 25 || man == 0) continue;
                const uint32_t q = man >> d;
                const uint32_t rem = man & ((1u << d) - 1u);
                const uint32_t half = d > 0 ? 1u << (d - 1) : 0u;
                csum += q + ((d > 0 && rem > half) ? 1u : 0u);
                tie |= d > 0 && rem == half;
            }
            csum = min(__reduce_add_sync(0xffffffffu, csum), 0x7FFFFFFFu);
            const bool any_tie = __any_sync(0xffffffffu, tie);
            if (lane == 0) blk_sum[b] = csum | (any_tie ? 0x80000000u : 0u);
        }
        __syncthreads();
        if (warp == 0) {
            // walk the blocks in order; stop at a half-way case or a carry into
            // the next binade and replay that block with real additions
            uint32_t m = m0;
            uint32_t ev_blk = 0xFFFFFFFFu;
            for (uint32_t b0 = b_first; b0 < nblk && ev_blk == 0xFFFFFFFFu; b0 += 32) {
                const uint32_t b = b0 + lane;
                const uint32_t raw = b < nblk ? blk_sum[b] : 0u;
                // any block sum >= 2^24 is a carry by itself; clamping keeps the scan inside 32 bits
                uint32_t inc = min(raw & 0x7FFFFFFFu, 1u << 25);
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += t;
                }
                const bool ev = (raw & 0x80000000u) || (m + inc >= (1u << 24));
                const uint32_t evm = __ballot_sync(0xffffffffu, ev);
                if (evm) {
                    const int l = __ffs(evm) - 1;
                    const uint32_t before = l == 0 ? 0u : __shfl_sync(0xffffffffu, inc, l - 1);
                    m += before;
                    ev_blk = b0 + l;
                } else {
                    m += __shfl_sync(0xffffffffu, inc, 31);
                }
            }
            float s_new = __uint_as_float((uint32_t) max(e_s - 23, 0) << 23) * (float) m;// exact: m < 2^24
            if (e_s < 24) s_new = ldexpf((float) m, e_s - 150);
            if (ev_blk != 0xFFFFFFFFu) {
                uint32_t keys[8];
                load_keys(work, ev_blk * kBlk, lane, keys);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t j = ev_blk * kBlk + lane * 8 + e;
                    sm.blk_terms[lane * 8 + e] = (keys[e] == 0 || j < pos) ? 0.f : term_of(val_of(keys[e]), M, T);
                }
                __syncwarp();
                if (lane == 0) {
                    for (int i = 0; i < kBlk; ++i) s_new = __fadd_rn(s_new, sm.blk_terms[i]);
                }
            }
            if (lane == 0) {
                sm.s = s_new;
                sm.pos = ev_blk == 0xFFFFFFFFu ? npad : (ev_blk + 1) * kBlk;
                sm.done = ev_blk == 0xFFFFFFFFu || (ev_blk + 1) >= nblk;
            }
        }
        __syncthreads();
    }

    stamp();// 6: denominator
    if (a.debug && tid == 0) a.debug[(int64_t) row * kDebugStride + 129 + 15] = (float) pass;
    // ---- probabilities of the top-k, top-p cut and the pick ------------------
    if (warp == 0) {
        const float S = sm.s;
        for (int i = lane; i < k; i += 32) {
            sm.top_term[i] = f16_to_f32(f32_to_f16_ref(__fdiv_rn(sm.top_term[i], S)));
        }
        __syncwarp();
        if (lane == 0) {
            if (a.debug) {
                a.debug[(int64_t) row * kDebugStride] = S;
                for (int i = 0; i < k && i < kSlots; ++i) {
                    a.debug[(int64_t) row * kDebugStride + 1 + i] = __uint_as_float(sm.top_idx[i]);
                    a.debug[(int64_t) row * kDebugStride + 1 + kSlots + i] = sm.top_term[i];
                }
            }
            pick_from_topk(sm.top_term, sm.top_idx, k, a.topp, random_val, a.result + (int64_t) row * a.result_stride);
        }
    }
}

}// namespace

namespace b200 {

}// namespace b200

namespace {

// Argmax branch (topp == 0 or topk <= 1; reference random_sample.cc:130-153: the first index among
// equal maxima) for rows that start on a 16-byte boundary.  A cluster of two CTAs per row, each streams
// one half with eight 128-bit loads in flight per thread; a thread only keeps the largest value it has
// seen (packed fp16 maxima) and the first vector that reached it, so the pass costs about one
// instruction per element; the winning vector is looked at again to name the element.
constexpr int kArgmaxThreads = 512;

__device__ __forceinline__ unsigned long long shfl_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    return v;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kArgmaxThreads) random_sample_argmax_kernel(RandomSampleArgs a) {
    namespace cg = cooperative_groups;
    __shared__ unsigned long long red[kArgmaxThreads / 32];
    __shared__ unsigned long long peer_best;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank();
    const int row = blockIdx.x >> 1, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint16_t *logits = a.logits + (int64_t) row * a.logits_stride;
    const uint32_t n = (uint32_t) a.voc, nvec = (n + 7) / 8;   // the last vector may be ragged
    const uint32_t half = (nvec + 1) / 2;
    const uint32_t v_begin = rank == 0 ? 0u : half, v_end = rank == 0 ? half : nvec;

    uint32_t best_key = 0, best_vec = 0xFFFFFFFFu;// key 0: nothing seen
    constexpr int kInFlight = 8;
    for (uint32_t v0 = v_begin + tid; v0 < v_end; v0 += kArgmaxThreads * kInFlight) {
        uint4 q[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t v = v0 + u * kArgmaxThreads;
            q[u] = make_uint4(0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u);
            if (v < v_end) {
                if (v * 8 + 8 <= n) {
                    q[u] = ld_stream(logits + (uint64_t) v * 8);
                } else {// ragged end of the row: element-wise, padded with -inf (never wins over a real element before it)
                    uint16_t h[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) h[e] = v * 8 + e < n ? logits[(uint64_t) v * 8 + e] : (uint16_t) 0xFC00;
                    q[u] = make_uint4(h[0] | ((uint32_t) h[1] << 16), h[2] | ((uint32_t) h[3] << 16),
                                      h[4] | ((uint32_t) h[5] << 16), h[6] | ((uint32_t) h[7] << 16));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t v = v0 + u * kArgmaxThreads;
            if (v < v_end) {
                const __half2 m2 = __hmax2(__hmax2(*reinterpret_cast<const __half2 *>(&q[u].x), *reinterpret_cast<const __half2 *>(&q[u].y)),
                                           __hmax2(*reinterpret_cast<const __half2 *>(&q[u].z), *reinterpret_cast<const __half2 *>(&q[u].w)));
                const uint32_t key = key_of(__half_as_ushort(__hmax(__low2half(m2), __high2half(m2))));
                if (key > best_key) {// strictly larger: the first vector that reaches the maximum stays
                    best_key = key;
                    best_vec = v;
                }
            }
        }
    }
    // (key, lowest vector) -> one 64-bit value whose maximum is the answer
    unsigned long long best = ((unsigned long long) best_key << 32) | (0xFFFFFFFFu - best_vec);
    best = shfl_max_u64(best);
    if (lane == 0) red[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = lane < kArgmaxThreads / 32 ? red[lane] : 0ull;
        best = shfl_max_u64(best);
        if (rank == 1 && lane == 0) *cluster.map_shared_rank(&peer_best, 0) = best;
    }
    cluster.sync();
    if (rank == 0 && warp == 0) {
        const unsigned long long other = peer_best;
        if (other > best) best = other;
        const uint32_t key = (uint32_t) (best >> 32), vec = 0xFFFFFFFFu - (uint32_t) (best & 0xFFFFFFFFu);
        // the first element of that vector whose key is the maximum
        uint32_t pos = 0xFFFFFFFFu;
        if (lane < 8) {
            const uint32_t i = vec * 8 + lane;
            if (i < n && key_of(logits[i]) == key) pos = i;
        }
        pos = __reduce_min_sync(0xffffffffu, pos);
        if (pos == 0xFFFFFFFFu) pos = 0;// only a row of NaNs gets here; the reference answers 0 for it
        if (lane == 0) a.result[(int64_t) row * a.result_stride] = pos;
    }
}

}// namespace

namespace b200 {

uint64_t random_sample_work_pitch(int voc) { return ((uint64_t) voc + kBlk - 1) / kBlk * kBlk; }

uint64_t random_sample_workspace_bytes(int voc, int rows) {
    return random_sample_work_pitch(voc) * 2ull * (uint64_t) rows + 256;
}

// True when this call will run the kernel that keeps the rows' working copies in the workspace (rows too long for
// the cluster's shared memory, or that kernel asked for through infiniopExtSelectKernel).
bool random_sample_uses_workspace(const RandomSampleArgs &a) {
    const bool sampling = a.topp > 0.f && a.topk > 1;
    return sampling && !(random_sample_pair_supported(a.voc) && kernel_choice(kFamilyRandomSample) != 1);
}

infiniopStatus_t random_sample_launch(const RandomSampleArgs &args_in, int rows, void *workspace,
                                      uint64_t workspace_size, cudaStream_t st) {
    RandomSampleArgs a = args_in;
    const bool sampling = a.topp > 0.f && a.topk > 1;
    if (sampling) {
        const int k = a.topk > a.voc ? a.voc : a.topk;
        if (k > kSlots) {
            fprintf(stderr, "infiniop[b200]: random sample supports topk <= %d (got %d)\n", kSlots, a.topk);
            return STATUS_BAD_PARAM;
        }
        if (!(a.temperature > 0.f)) return STATUS_BAD_PARAM;
        // Rows that fit the shared memory of a cluster never touch the workspace.
        if (!random_sample_uses_workspace(a)) return random_sample_pair_launch(a, rows, st);
        if (workspace == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
        if (workspace_size < random_sample_workspace_bytes(a.voc, rows)) return STATUS_INSUFFICIENT_WORKSPACE;
        a.work = reinterpret_cast<uint16_t *>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t) 255);
        a.work_pitch = (int64_t) random_sample_work_pitch(a.voc);
    }
    if (!sampling && aligned16(a.logits) && a.logits_stride % 8 == 0 && a.voc >= 1) {
        random_sample_argmax_kernel<<<2 * rows, kArgmaxThreads, 0, st>>>(a);
        return check_launch("random_sample_argmax");
    }
    const uint32_t nblk = (uint32_t) ((a.voc + kBlk - 1) / kBlk);
    const size_t smem = sizeof(Shared) + (size_t) nblk * sizeof(uint32_t);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(random_sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) !=
            cudaSuccess) {
            cudaGetLastError();
            return STATUS_BAD_PARAM;// vocabulary too large for the per-block table
        }
    }
    random_sample_kernel<<<rows, kThreads, smem, st>>>(a);
    return check_launch("random_sample");
}

}// namespace b200

INFINIOP_API infiniopStatus_t infiniopCreateRandomSampleDescriptor(infiniopHandle_t handle,
                                                                   infiniopRandomSampleDescriptor_t *desc_ptr,
                                                                   infiniopTensorDescriptor_t result,
                                                                   infiniopTensorDescriptor_t probs) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (result == nullptr || probs == nullptr) return STATUS_BAD_PARAM;
    // Checks and codes of reference random_sample_cuda.cc:9-19 and of the CPU
    // backend (random_sample.cc:10-23), which also insists on fp16 logits.
    if (probs->ndim != 1) return STATUS_BAD_TENSOR_SHAPE;
    if (!dt_eq(probs->dt, F16)) return STATUS_BAD_TENSOR_DTYPE;
    if (!dt_eq(result->dt, U64)) return STATUS_BAD_TENSOR_DTYPE;
    if (result->ndim != 1 && result->shape[0] != 1) return STATUS_BAD_TENSOR_SHAPE;
    if (probs->strides[0] != 1) return STATUS_BAD_TENSOR_STRIDES;
    if (probs->shape[0] == 0 || probs->shape[0] > 0x7FFFFFFFull) return STATUS_BAD_TENSOR_SHAPE;
    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow)
        RandomSampleDesc{DevNvGpu, h->device_id, h->sm_count, (int) probs->shape[0], (int) result->shape[0]};
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    *desc_ptr = reinterpret_cast<infiniopRandomSampleDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetRandomSampleWorkspaceSize(infiniopRandomSampleDescriptor_t desc,
                                                                   uint64_t *size) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = random_sample_workspace_bytes(reinterpret_cast<RandomSampleDesc *>(desc)->voc, 1);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopRandomSample(infiniopRandomSampleDescriptor_t desc, void *workspace,
                                                   uint64_t workspace_size, void *result, void const *probs,
                                                   float random_val, float topp, int topk, float temperature,
                                                   void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (result == nullptr || probs == nullptr) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<RandomSampleDesc *>(desc);
    DeviceGuard guard(d->device_id);
    RandomSampleArgs a{};
    a.logits = reinterpret_cast<const uint16_t *>(probs);
    a.logits_stride = 0;
    a.result = reinterpret_cast<uint64_t *>(result);
    a.result_stride = 0;
    a.random_vals = nullptr;
    a.random_val = random_val;
    a.topp = topp;
    a.topk = topk;
    a.temperature = temperature;
    a.voc = d->voc;
    a.debug = nullptr;
    return random_sample_launch(a, 1, workspace, workspace_size, reinterpret_cast<cudaStream_t>(stream));
}

INFINIOP_API infiniopStatus_t infiniopDestroyRandomSampleDescriptor(infiniopRandomSampleDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<RandomSampleDesc *>(desc);
    return STATUS_SUCCESS;
}

// ---- batched extension (include/infiniop_ext.h) -------------------------------

#include "../../include/infiniop_ext.h"

INFINIOP_API infiniopStatus_t infiniopGetRandomSampleBatchWorkspaceSize(infiniopRandomSampleDescriptor_t desc,
                                                                        uint64_t rows, uint64_t *size) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (size == nullptr || rows == 0 || rows > 0x7FFFFFFFull) return STATUS_BAD_PARAM;
    *size = random_sample_workspace_bytes(reinterpret_cast<RandomSampleDesc *>(desc)->voc, (int) rows);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopRandomSampleBatchTrace(infiniopRandomSampleDescriptor_t desc, void *workspace,
                                                             uint64_t workspace_size, void *results,
                                                             void const *logits, int64_t row_stride, uint64_t rows,
                                                             void const *random_vals, float topp, int topk,
                                                             float temperature, void *trace, void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (results == nullptr || logits == nullptr || random_vals == nullptr) return STATUS_BAD_PARAM;
    if (rows == 0) return STATUS_SUCCESS;
    if (rows > 0x7FFFFFFFull) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<RandomSampleDesc *>(desc);
    DeviceGuard guard(d->device_id);
    RandomSampleArgs a{};
    a.logits = reinterpret_cast<const uint16_t *>(logits);
    a.logits_stride = row_stride;
    a.result = reinterpret_cast<uint64_t *>(results);
    a.result_stride = 1;
    a.random_vals = reinterpret_cast<const float *>(random_vals);
    a.random_val = 0.f;
    a.topp = topp;
    a.topk = topk;
    a.temperature = temperature;
    a.voc = d->voc;
    a.debug = reinterpret_cast<float *>(trace);
    return random_sample_launch(a, (int) rows, workspace, workspace_size, reinterpret_cast<cudaStream_t>(stream));
}

INFINIOP_API infiniopStatus_t infiniopRandomSampleBatch(infiniopRandomSampleDescriptor_t desc, void *workspace,
                                                        uint64_t workspace_size, void *results, void const *logits,
                                                        int64_t row_stride, uint64_t rows, void const *random_vals,
                                                        float topp, int topk, float temperature, void *stream) {
    return infiniopRandomSampleBatchTrace(desc, workspace, workspace_size, results, logits, row_stride, rows,
                                          random_vals, topp, topk, temperature, nullptr, stream);
}

// ---- batched sampling of vocabulary-sharded rows over peer memory, one launch --------
//
// The exchange of peer_exchange.cu folded into the sampling kernel: its CTAs wait for the peers' "shard is final"
// words, read their row out of the `world` shards with peer loads, and the thread that picks a row's index stores it
// into every rank's result array; the row that finishes last runs the "done" round.  Same flag words and call
// counter as infiniopExtPeerGatherRows / infiniopExtPeerPublishResults, so a rank without rows of its own takes part
// with those two (nrows = 0).  Conditions: the sampling branch (topp > 0, 2 <= topk <= 64), rows of at most 262144
// logits, equal shards of a multiple of 8 columns; otherwise STATUS_BAD_PARAM and the three-launch form applies.
INFINIOP_API infiniopStatus_t infiniopRandomSampleBatchPeer(infiniopRandomSampleDescriptor_t desc, void *const *results,
                                                            void *const *shards, const int64_t *shard_row_strides,
                                                            uint64_t shard_cols, void *const *flags, uint32_t world,
                                                            uint32_t rank, uint64_t row0, uint64_t nrows,
                                                            void const *random_vals, float topp, int topk,
                                                            float temperature, void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    auto *d = reinterpret_cast<RandomSampleDesc *>(desc);
    if (results == nullptr || shards == nullptr || shard_row_strides == nullptr || flags == nullptr || random_vals == nullptr) {
        return STATUS_BAD_PARAM;
    }
    if (world == 0 || world > kPeerMaxRanks || rank >= world || nrows == 0 || nrows > 0x7FFFFFull) return STATUS_BAD_PARAM;
    const int k = topk > d->voc ? d->voc : topk;
    if (!(topp > 0.f) || topk < 2 || k > kSlots || !(temperature > 0.f)) return STATUS_BAD_PARAM;
    if (!random_sample_pair_supported(d->voc) || kernel_choice(kFamilyRandomSample) == 1) return STATUS_BAD_PARAM;
    if (shard_cols == 0 || shard_cols % 8 != 0 || shard_cols * world != (uint64_t) d->voc) return STATUS_BAD_PARAM;
    RandomSampleArgs a{};
    a.random_vals = reinterpret_cast<const float *>(random_vals);
    a.topp = topp, a.topk = topk, a.temperature = temperature, a.voc = d->voc;
    a.peer.world = world, a.peer.rank = rank, a.peer.shard_vecs = (uint32_t) (shard_cols / 8);
    a.peer.rows = (uint32_t) nrows, a.peer.row0 = row0;
    for (uint32_t r = 0; r < world; ++r) {
        if (results[r] == nullptr || shards[r] == nullptr || flags[r] == nullptr || !aligned16(shards[r]) ||
            shard_row_strides[r] % 8 != 0) {
            return STATUS_BAD_PARAM;
        }
        a.peer.shard[r] = reinterpret_cast<const uint16_t *>(shards[r]);
        a.peer.shard_stride[r] = shard_row_strides[r];
        a.peer.flags[r] = reinterpret_cast<uint32_t *>(flags[r]);
        a.peer.results[r] = reinterpret_cast<unsigned long long *>(results[r]);
    }
    a.logits = a.peer.shard[rank];// unused by the sharded load; kept non-null
    a.logits_stride = shard_row_strides[rank];
    a.result = reinterpret_cast<uint64_t *>(results[rank]) + row0;
    a.result_stride = 1;
    DeviceGuard guard(d->device_id);
    return random_sample_pair_launch(a, (int) nrows, reinterpret_cast<cudaStream_t>(stream));
}

// ---- batched sampling without a caller-provided workspace -----------------------
//
// Some hosts of this library may not allocate device memory at the point where
// they sample: a serving loop that has handed every byte of HBM to its own KV
// cache / arena allocator and has no workspace slab to lend, or a plug-in that
// is only given input and output pointers.  For them the working copy of the
// rows lives in a fixed array inside the library image.  Every GPU that loads
// the library carries these 32 MiB until the process exits.
constexpr uint64_t kStaticScratchBytes = 32ull << 20;
static __device__ __align__(256) unsigned char g_sample_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
// Device address of g_sample_scratch per device ordinal, published with a release store once it is known.
// Two host threads that make the first call on a device together both look the address up and store the same
// value; nobody reads a half-written entry.
std::atomic<void *> g_scratch_addr[kMaxDevices];
}// namespace

INFINIOP_API infiniopStatus_t infiniopRandomSampleBatchStatic(infiniopRandomSampleDescriptor_t desc, void *results,
                                                              void const *logits, int64_t row_stride, uint64_t rows,
                                                              void const *random_vals, float topp, int topk,
                                                              float temperature, void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (results == nullptr || logits == nullptr || random_vals == nullptr) return STATUS_BAD_PARAM;
    if (rows == 0) return STATUS_SUCCESS;
    auto *d = reinterpret_cast<RandomSampleDesc *>(desc);
    if (d->device_id < 0 || d->device_id >= kMaxDevices) return STATUS_BAD_DEVICE;
    if (rows > 0x7FFFFFFFull) return STATUS_BAD_PARAM;
    RandomSampleArgs a{};
    a.logits = reinterpret_cast<const uint16_t *>(logits);
    a.logits_stride = row_stride;
    a.result = reinterpret_cast<uint64_t *>(results);
    a.result_stride = 1;
    a.random_vals = reinterpret_cast<const float *>(random_vals);
    a.random_val = 0.f;
    a.topp = topp;
    a.topk = topk;
    a.temperature = temperature;
    a.voc = d->voc;
    a.debug = nullptr;
    // The size limit binds only the kernel that keeps its working copies in the array (rows of more than
    // 262144 logits); shorter rows are sampled out of shared memory and use no scratch at all.
    if (random_sample_uses_workspace(a) && random_sample_workspace_bytes(d->voc, (int) rows) > kStaticScratchBytes) {
        fprintf(stderr,
                "infiniop[b200]: infiniopRandomSampleBatchStatic: %llu rows of %d logits need %llu bytes of scratch, "
                "the built-in array holds %llu; use infiniopRandomSampleBatch with a workspace\n",
                (unsigned long long) rows, d->voc, (unsigned long long) random_sample_workspace_bytes(d->voc, (int) rows),
                (unsigned long long) kStaticScratchBytes);
        return STATUS_INSUFFICIENT_WORKSPACE;
    }
    DeviceGuard guard(d->device_id);
    void *scratch = g_scratch_addr[d->device_id].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        // The array's name is only a host-side handle; the kernel needs the
        // address the array has on THIS device, asked for once per device with
        // that device current (the guard above made it so).
        cudaError_t e = cudaGetSymbolAddress(&scratch, g_sample_scratch);
        if (e != cudaSuccess || scratch == nullptr) {
            fprintf(stderr, "infiniop[b200]: cudaGetSymbolAddress(g_sample_scratch) failed: %s\n", cudaGetErrorString(e));
            cudaGetLastError();
            return STATUS_EXECUTION_FAILED;
        }
        g_scratch_addr[d->device_id].store(scratch, std::memory_order_release);
    }
    return random_sample_launch(a, (int) rows, scratch, kStaticScratchBytes, reinterpret_cast<cudaStream_t>(stream));
}
