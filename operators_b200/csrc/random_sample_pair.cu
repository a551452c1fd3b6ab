// Random sample, shared-memory resident form: a thread-block cluster of two
// CTAs owns one row of up to 131072 logits.
//
// Same result as random_sample_kernel (random_sample.cu), i.e. the index the
// reference CPU backend returns (src/ops/random_sample/cpu/random_sample.cc:
// 45-129); see that file's header for the three facts the algorithm rests on
// (streaming insertion, closed form of the permuted row, binade-wise integer
// sum).  What differs is where the row lives and how the work is spread:
//
//  * The row is read from HBM exactly once and kept in shared memory as 16-bit
//    order-preserving keys: the leader CTA holds elements [0, 65536), the helper
//    the rest.  Every later step (candidate search, record patches, block sums)
//    runs on shared memory; the two CTAs exchange a few hundred bytes through
//    distributed shared memory and meet at hardware cluster barriers (no
//    flag spinning anywhere).
//  * The denominator is formed for FOUR binades of the running sum at once:
//    per element z = 2*term/ulp0 comes from the special-function unit
//    (ex2.approx), floor(z) gives round-to-nearest(term/ulp_d) for d = 0..3 with
//    shifts, and only elements whose z lies within the approximation's error
//    band of an integer (or that are very large) are re-evaluated exactly with
//    a double-precision exp, densely, by the whole CTA.  The walk over the
//    256-element block sums switches level when the running sum carries into
//    the next binade, after replaying that one block with real fp32 additions.
#include "common.cuh"
#include "random_sample.cuh"
#include "random_sample_device.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;
using namespace b200;

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kBlk = 256;
constexpr int kListCap = 64;      // per-warp ordered list
constexpr int kFlatCap = 1024;    // per-CTA ordered list (candidates, flagged records)
constexpr int kHalfElems = 65536; // keys held by one CTA
constexpr int kMaxBlk = 2 * kHalfElems / kBlk;
constexpr int kLevels = 4;
constexpr int kUncCap = 6144;
constexpr int kMaxRounds = 6;     // 6 x 4 binades covers any sum of <= 2^17 terms <= 1
constexpr uint32_t kEmptyMin = 0xFFFFFFFFu;

struct WarpLists {
    uint32_t idx[kWarps][kListCap];
    uint16_t key[kWarps][kListCap];
    int cnt[kWarps];
    int overflow;
};
struct FlatList {
    uint32_t idx[kFlatCap];
    uint16_t key[kFlatCap];
    int cnt;
    int overflow;
};
struct Mail {// written by the other CTA of the pair (the leader also fills its own copy)
    uint32_t L_peer;
    uint32_t tau_mid;
    uint32_t mkey;
    float s_base;
    uint32_t pos_base;
    int done;
};
struct Aux {
    WarpLists wl;
    FlatList own;
    FlatList peer;// leader: copy of the helper's list
    uint32_t top_key[kSlots];
    uint32_t top_idx[kSlots];
    float top_term[kSlots];
    float blk_terms[kBlk];
    uint32_t C[kLevels][kMaxBlk];// integer block sums per binade level
    uint32_t tie[kMaxBlk];       // bit d: block holds an exact half-way case at level d
    uint32_t unc[kUncCap];       // positions (local) to re-evaluate exactly
    int unc_cnt;
    Mail mail;
};

constexpr size_t kSmemBytes = (size_t) kHalfElems * 2 + sizeof(Aux);

__device__ __forceinline__ void lds_keys(const uint16_t *p, uint32_t keys[8]) {
    const uint4 v = *reinterpret_cast<const uint4 *>(p);
    const uint32_t *w = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        keys[2 * k] = w[k] & 0xFFFFu;
        keys[2 * k + 1] = w[k] >> 16;
    }
}

// Ordered append of the flagged elements of one block to this warp's list.
__device__ __forceinline__ void warp_append(WarpLists &wl, int warp, int lane, uint32_t mask, const uint32_t keys[8],
                                            uint32_t base_idx) {
    const uint32_t any = __ballot_sync(0xffffffffu, mask != 0);
    if (any == 0) return;
    const int cnt = __popc(mask);
    int pre = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, pre, o);
        if (lane >= o) pre += t;
    }
    const int total = __shfl_sync(0xffffffffu, pre, 31);
    const int start = wl.cnt[warp];
    if (start + total > kListCap) {
        if (lane == 0) wl.overflow = 1;
    } else {
        int at = start + pre - cnt;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (mask & (1u << e)) {
                wl.idx[warp][at] = base_idx + lane * 8 + e;
                wl.key[warp][at] = (uint16_t) keys[e];
                ++at;
            }
        }
    }
    __syncwarp();
    if (lane == 0) wl.cnt[warp] = min(start + total, kListCap + 1);
    __syncwarp();
}

// Warp lists -> one ordered list (warp 0 of the CTA calls it).
__device__ __forceinline__ void flatten(const WarpLists &wl, FlatList &fl, int lane) {
    int total = 0;
    bool over = wl.overflow != 0;
    for (int w = 0; w < kWarps && !over; ++w) {
        const int c = wl.cnt[w];
        if (total + c > kFlatCap) {
            over = true;
            break;
        }
        for (int i = lane; i < c; i += 32) {
            fl.idx[total + i] = wl.idx[w][i];
            fl.key[total + i] = wl.key[w][i];
        }
        total += c;
    }
    __syncwarp();
    if (lane == 0) {
        fl.cnt = over ? 0 : total;
        fl.overflow = over ? 1 : 0;
    }
}

struct MinBuf {
    uint32_t v0, v1, tau;
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

// One warp walks a 256-element block (local or the peer's shared memory) in
// index order and feeds every element above the running k-th largest value;
// a record is overwritten with that value.
__device__ __forceinline__ void records_direct_block(uint16_t *blk, uint32_t first_in_blk, int lane, MinBuf &m) {
    uint32_t keys[8];
    lds_keys(blk + lane * 8, keys);
    uint32_t mask = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        if ((uint32_t) (lane * 8 + e) >= first_in_blk && keys[e] > m.tau) mask |= 1u << e;
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
            if (lane == 0) blk[src * 8 + e] = (uint16_t) m.tau;
            minbuf_replace(m, lane, key);
        }
        if (lane == src) mask &= mask - 1;
        any = __ballot_sync(0xffffffffu, mask != 0);
    }
}

// Exact contribution of one term to the block sums of all levels.
__device__ __forceinline__ void exact_contrib(Aux &ax, uint32_t blk, float v, float M, float T, int e0) {
    const uint32_t tb = __float_as_uint(term_of(v, M, T));
    int e_t = (int) ((tb >> 23) & 0xFFu);
    uint32_t man = tb & 0x7FFFFFu;
    if (e_t == 0) e_t = 1;
    else man |= 0x800000u;
    if (man == 0) return;
    uint32_t ties = 0;
#pragma unroll
    for (int d = 0; d < kLevels; ++d) {
        const int sh = e0 + d - e_t;// >= 0: every term is <= 1 <= running sum
        if (sh >= 25) continue;
        const uint32_t q = man >> sh;
        const uint32_t rem = man & ((1u << sh) - 1u);
        const uint32_t half = sh > 0 ? 1u << (sh - 1) : 0u;
        const uint32_t c = q + ((sh > 0 && rem > half) ? 1u : 0u);
        if (c) atomicAdd(&ax.C[d][blk], c);
        if (sh > 0 && rem == half) ties |= 1u << d;
    }
    if (ties) atomicOr(&ax.tie[blk], ties);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) random_sample_pair_kernel(RandomSampleArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint16_t *keys = reinterpret_cast<uint16_t *>(smem_raw);
    Aux &ax = *reinterpret_cast<Aux *>(smem_raw + (size_t) kHalfElems * 2);
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank();
    const bool leader = rank == 0;
    uint16_t *peer_keys = cluster.map_shared_rank(keys, rank ^ 1u);
    Aux *peer_ax = cluster.map_shared_rank(&ax, rank ^ 1u);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x >> 1;
    const uint32_t n = (uint32_t) a.voc;
    const uint32_t n0 = min(n, (uint32_t) kHalfElems);           // leader's elements
    const uint32_t my_base = leader ? 0u : (uint32_t) kHalfElems;// helper starts at 65536 (only used when n > 65536)
    const uint32_t my_n = leader ? n0 : n - n0;
    const uint32_t my_nblk = (my_n + kBlk - 1) / kBlk;
    const uint32_t my_pad = my_nblk * kBlk;
    const uint32_t nblk0 = (n0 + kBlk - 1) / kBlk;
    const uint32_t nblk = nblk0 + (n - n0 + kBlk - 1) / kBlk;
    const uint16_t *logits = a.logits + (int64_t) row * a.logits_stride + my_base;
    const float random_val = a.random_vals ? a.random_vals[row] : a.random_val;
    const float T = a.temperature;
    const int k = a.topk > (int) n ? (int) n : a.topk;

    const long long t_entry = clock64();
    int stamp_i = 0;
    auto stamp = [&]() {
        if (a.debug && leader && tid == 0 && stamp_i < 15) {
            a.debug[(int64_t) row * kDebugStride + 129 + stamp_i] = (float) (clock64() - t_entry);
        }
        ++stamp_i;
    };

    // ---- P1: logits -> keys in shared memory; per-thread maxima -------------------------
    const bool in_aligned = (reinterpret_cast<uintptr_t>(logits) & 15u) == 0;
    uint32_t tmax = 0;
    constexpr int kInFlight = 8;
    for (uint32_t base0 = tid * 8; base0 < my_pad; base0 += kThreads * 8 * kInFlight) {
        uint4 raw[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t base = base0 + u * kThreads * 8;
            if (in_aligned && base + 8 <= my_n) raw[u] = ld_stream(logits + base);
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t base = base0 + u * kThreads * 8;
            if (base >= my_pad) break;
            uint32_t kk[8];
            if (in_aligned && base + 8 <= my_n) {
                const uint32_t *p = reinterpret_cast<const uint32_t *>(&raw[u]);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    kk[2 * q] = key_of((uint16_t) (p[q] & 0xFFFFu));
                    kk[2 * q + 1] = key_of((uint16_t) (p[q] >> 16));
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) kk[e] = base + e < my_n ? key_of(logits[base + e]) : 0u;
            }
            uint4 o;
            o.x = kk[0] | (kk[1] << 16);
            o.y = kk[2] | (kk[3] << 16);
            o.z = kk[4] | (kk[5] << 16);
            o.w = kk[6] | (kk[7] << 16);
            *reinterpret_cast<uint4 *>(keys + base) = o;
#pragma unroll
            for (int e = 0; e < 8; ++e) tmax = max(tmax, kk[e]);
        }
    }
    if (tid < kWarps) ax.wl.cnt[tid] = 0;
    if (tid == 0) {
        ax.wl.overflow = 0;
        ax.unc_cnt = 0;
    }
    // local lower bound of the k-th largest key: k-th largest per-thread maximum
    uint32_t L_mine = 0;
    {
        const int have = __syncthreads_count(tmax >= 1);
        if (have > 0) {// uniform
            const int need = k < have ? k : have;
            uint32_t lo = 1, hi = 65535;
            while (lo < hi) {
                const uint32_t mid = (lo + hi + 1) >> 1;
                if (__syncthreads_count(tmax >= mid) >= need) lo = mid;
                else hi = mid - 1;
            }
            L_mine = have < k ? 1u : lo;
        }
    }
    if (tid == 0) peer_ax->mail.L_peer = L_mine;
    cluster.sync();// CS1
    stamp();       // 0: keys resident
    const uint32_t L = max(max(L_mine, ax.mail.L_peer), 1u);

    // ---- P2: candidates (key >= L), ordered --------------------------------------------
    auto scan_blocks = [&](uint32_t blk_begin, uint32_t blk_end, uint32_t thresh, bool strict) {
        // all warps of this CTA: blocks [blk_begin, blk_end) of the LOCAL half, contiguous span per warp
        const uint32_t cnt = blk_end - blk_begin;
        const uint32_t span = (cnt + kWarps - 1) / kWarps;
        const uint32_t b0 = blk_begin + warp * span, b1 = min(blk_end, b0 + span);
        for (uint32_t b = b0; b < b1; ++b) {
            uint32_t kk[8];
            lds_keys(keys + b * kBlk + lane * 8, kk);
            uint32_t mask = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e) mask |= ((strict ? kk[e] > thresh : kk[e] >= thresh) ? 1u : 0u) << e;
            warp_append(ax.wl, warp, lane, mask, kk, my_base + b * kBlk);
        }
    };
    scan_blocks(0, my_nblk, L, false);
    __syncthreads();
    if (warp == 0) flatten(ax.wl, ax.own, lane);
    __syncthreads();
    if (!leader) {
        for (int i = tid; i < ax.own.cnt; i += kThreads) {
            peer_ax->peer.idx[i] = ax.own.idx[i];
            peer_ax->peer.key[i] = ax.own.key[i];
        }
        if (tid == 0) {
            peer_ax->peer.cnt = ax.own.cnt;
            peer_ax->peer.overflow = ax.own.overflow;
        }
    }
    cluster.sync();// CS2
    stamp();       // 1: candidate lists at the leader

    // ---- P3 (leader): exact top-k, records of the leader half --------------------------
    MinBuf mb{kEmptyMin, kEmptyMin, 0};
    float M = 0.f;
    if (leader) {
        if (warp == 0) {
            TopBuf tb{0, 0, 0, 0};
            if (!ax.own.overflow && !ax.peer.overflow) {
                for (int c = 0; c < ax.own.cnt; ++c) topbuf_insert(tb, lane, k, ax.own.key[c], ax.own.idx[c]);
                for (int c = 0; c < ax.peer.cnt; ++c) topbuf_insert(tb, lane, k, ax.peer.key[c], ax.peer.idx[c]);
            } else {
                // more ties than the lists hold: stream the whole row
                for (uint32_t b = 0; b < nblk; ++b) {
                    const uint16_t *blk = b < nblk0 ? keys + b * kBlk : peer_keys + (b - nblk0) * kBlk;
                    const uint32_t gbase = b < nblk0 ? b * kBlk : (uint32_t) kHalfElems + (b - nblk0) * kBlk;
                    uint32_t kk[8];
                    lds_keys(blk + lane * 8, kk);
                    const uint32_t kth = __shfl_sync(0xffffffffu, (k - 1) < 32 ? tb.k0 : tb.k1, (k - 1) & 31);
                    uint32_t mask = 0;
#pragma unroll
                    for (int e = 0; e < 8; ++e) mask |= (kk[e] > kth ? 1u : 0u) << e;
                    uint32_t any = __ballot_sync(0xffffffffu, mask != 0);
                    while (any) {
                        const int src = __ffs(any) - 1;
                        const uint32_t smask = __shfl_sync(0xffffffffu, mask, src);
                        const int e = __ffs(smask) - 1;
                        uint32_t key = 0;
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            if (t == e) key = kk[t];
                        }
                        key = __shfl_sync(0xffffffffu, key, src);
                        topbuf_insert(tb, lane, k, key, gbase + src * 8 + e);
                        if (lane == src) mask &= mask - 1;
                        any = __ballot_sync(0xffffffffu, mask != 0);
                    }
                }
            }
            ax.top_key[lane] = tb.k0;
            ax.top_key[lane + 32] = tb.k1;
            ax.top_idx[lane] = tb.i0;
            ax.top_idx[lane + 32] = tb.i1;
            __syncwarp();
            const float Mw = val_of(ax.top_key[0]);
            for (int i = lane; i < k; i += 32) ax.top_term[i] = term_of(val_of(ax.top_key[i]), Mw, T);
            __syncwarp();
            if (lane == 0) {
                float s = 0.f;
                for (int i = 0; i < k; ++i) s = __fadd_rn(s, ax.top_term[i]);
                ax.mail.s_base = s;
                ax.mail.pos_base = (uint32_t) k;
                ax.mail.mkey = ax.top_key[0];
                ax.mail.done = (uint32_t) k >= n;
            }
        }
        __syncthreads();
        stamp();// 2: top-k in order, top-k terms summed
        M = val_of(ax.mail.mkey);

        if ((uint32_t) k < n) {
            if (warp == 0) {
                if (lane < k) mb.v0 = keys[lane];
                if (lane + 32 < k) mb.v1 = keys[lane + 32];
                mb.tau = __reduce_min_sync(0xffffffffu, min(mb.v0, mb.v1));
            }
            const uint32_t head_blocks = min(nblk0, 8u);
            if (warp == 0) {
                for (uint32_t b = 0; b < head_blocks; ++b) {
                    records_direct_block(keys + b * kBlk, b == 0 ? (uint32_t) k : 0u, lane, mb);
                }
                if (lane == 0) ax.mail.tau_mid = mb.tau;
            }
            uint32_t t_begin = head_blocks;
            while (t_begin < nblk0) {
                const uint32_t t_end = min(nblk0, t_begin * 2);
                if (tid < kWarps) ax.wl.cnt[tid] = 0;
                if (tid == 0) ax.wl.overflow = 0;
                __syncthreads();
                scan_blocks(t_begin, t_end, ax.mail.tau_mid, true);
                __syncthreads();
                if (warp == 0) {
                    if (!ax.wl.overflow) {
                        for (int w = 0; w < kWarps; ++w) {
                            const int cnt = ax.wl.cnt[w];
                            for (int c = 0; c < cnt; ++c) {
                                const uint32_t key = ax.wl.key[w][c];
                                if (key > mb.tau) {
                                    if (lane == 0) keys[ax.wl.idx[w][c]] = (uint16_t) mb.tau;
                                    minbuf_replace(mb, lane, key);
                                }
                            }
                        }
                    } else {
                        for (uint32_t b = t_begin; b < t_end; ++b) records_direct_block(keys + b * kBlk, 0u, lane, mb);
                    }
                    if (lane == 0) ax.mail.tau_mid = mb.tau;
                }
                t_begin = t_end;
                __syncthreads();
            }
        }
        __syncthreads();
        if (tid == 0) {// hand the helper what it needs
            peer_ax->mail.tau_mid = ax.mail.tau_mid;
            peer_ax->mail.mkey = ax.mail.mkey;
            peer_ax->mail.s_base = ax.mail.s_base;
            peer_ax->mail.pos_base = ax.mail.pos_base;
            peer_ax->mail.done = ax.mail.done;
        }
    }
    cluster.sync();// CS3
    stamp();       // 3: leader half patched

    // ---- P4 (helper): elements of its half above the running k-th value -----------------
    if (!leader && my_n > 0 && !ax.mail.done) {
        if (tid < kWarps) ax.wl.cnt[tid] = 0;
        if (tid == 0) ax.wl.overflow = 0;
        __syncthreads();
        scan_blocks(0, my_nblk, ax.mail.tau_mid, true);
        __syncthreads();
        if (warp == 0) flatten(ax.wl, ax.own, lane);
        __syncthreads();
        for (int i = tid; i < ax.own.cnt; i += kThreads) {
            peer_ax->peer.idx[i] = ax.own.idx[i];
            peer_ax->peer.key[i] = ax.own.key[i];
        }
        if (tid == 0) {
            peer_ax->peer.cnt = ax.own.cnt;
            peer_ax->peer.overflow = ax.own.overflow;
        }
    }
    cluster.sync();// CS4

    // ---- P5 (leader, warp 0): records of the helper half -------------------------------
    if (leader && warp == 0 && n > n0 && !ax.mail.done) {
        if (!ax.peer.overflow) {
            for (int c = 0; c < ax.peer.cnt; ++c) {
                const uint32_t key = ax.peer.key[c];
                if (key > mb.tau) {
                    if (lane == 0) peer_keys[ax.peer.idx[c] - (uint32_t) kHalfElems] = (uint16_t) mb.tau;
                    minbuf_replace(mb, lane, key);
                }
            }
        } else {
            for (uint32_t b = 0; b < nblk - nblk0; ++b) records_direct_block(peer_keys + b * kBlk, 0u, lane, mb);
        }
    }
    cluster.sync();// CS5
    stamp();       // 4: whole row patched
    M = val_of(ax.mail.mkey);

    // ---- denominator rounds -------------------------------------------------------------
    const float A = kLog2e / T;
    int rounds = 0;
    for (int round = 0; round < kMaxRounds && !ax.mail.done; ++round) {
        ++rounds;
        const float s_base = ax.mail.s_base;
        const uint32_t pos = ax.mail.pos_base;
        const int e0 = (int) ((__float_as_uint(s_base) >> 23) & 0xFFu);
        const float scale = __uint_as_float((uint32_t) (151 - e0 + 127) << 23);// 2 / ulp(s_base), a power of two
        const float cut = -2.0f - (float) (151 - e0);                          // z < 1/4: no contribution at any level
        const float band = 6.0e-6f;                                            // > 2^-17.5, relative error bound of z
        const uint32_t gb_first = pos / kBlk;                                  // first global block still to sum
        const uint32_t lb_first = leader ? gb_first : (gb_first > nblk0 ? gb_first - nblk0 : 0u);
        // block b of the local half is global block b (+ nblk0 for the helper)
        const uint32_t goff = leader ? 0u : nblk0;
        if (tid == 0) ax.unc_cnt = 0;
        for (uint32_t i = lb_first + tid; i < my_nblk; i += kThreads) {
#pragma unroll
            for (int d = 0; d < kLevels; ++d) ax.C[d][i + goff] = 0;
            ax.tie[i + goff] = 0;
        }
        __syncthreads();
        if (lb_first < my_nblk) {
            const uint32_t cntb = my_nblk - lb_first;
            const uint32_t span = (cntb + kWarps - 1) / kWarps;
            const uint32_t b0 = lb_first + warp * span, b1 = min(my_nblk, b0 + span);
            for (uint32_t b = b0; b < b1; ++b) {
                uint32_t kk[8];
                lds_keys(keys + b * kBlk + lane * 8, kk);
                uint32_t F = 0, Bp = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t gpos = my_base + b * kBlk + lane * 8 + e;
                    if (kk[e] == 0 || gpos < pos) continue;
                    const float v = val_of(kk[e]);
                    const float arg = __fmul_rn(__fsub_rn(v, M), A);
                    if (arg < cut) continue;
                    const float z = fast_exp2(arg) * scale;
                    const float fz = floorf(z);
                    const float fr = z - fz;
                    if (fminf(fr, 1.0f - fr) <= z * band || z >= 1048576.0f) {
                        const int slot = atomicAdd(&ax.unc_cnt, 1);
                        if (slot < kUncCap) ax.unc[slot] = b * kBlk + lane * 8 + e;
                        else exact_contrib(ax, b + goff, v, M, T, e0);// list full: settle it here
                    } else {
                        const uint32_t f = (uint32_t) fz;
                        F += f;
                        Bp += ((f & 15u) * 0x00204081u) & 0x01010101u;// bit i of f -> byte i
                    }
                }
                F = __reduce_add_sync(0xffffffffu, F);
                const uint32_t lo = __reduce_add_sync(0xffffffffu, Bp & 0x00FF00FFu);       // bits 0 and 2
                const uint32_t hi = __reduce_add_sync(0xffffffffu, (Bp >> 8) & 0x00FF00FFu);// bits 1 and 3
                if (lane == 0) {
                    const uint32_t B0 = lo & 0xFFFFu, B2 = lo >> 16, B1 = hi & 0xFFFFu, B3 = hi >> 16;
                    // sum over elements of round(f_exact / 2^(d+1)) = sum (f >> (d+1)) + sum bit_d(f)
                    // (added, not stored: exact contributions of this block may already be there)
                    atomicAdd(&ax.C[0][b + goff], ((F - B0) >> 1) + B0);
                    atomicAdd(&ax.C[1][b + goff], ((F - B0 - 2 * B1) >> 2) + B1);
                    atomicAdd(&ax.C[2][b + goff], ((F - B0 - 2 * B1 - 4 * B2) >> 3) + B2);
                    atomicAdd(&ax.C[3][b + goff], ((F - B0 - 2 * B1 - 4 * B2 - 8 * B3) >> 4) + B3);
                }
            }
        }
        __syncthreads();
        {// exact re-evaluation of the uncertain elements, densely
            const int cnt = min(ax.unc_cnt, kUncCap);
            for (int i = tid; i < cnt; i += kThreads) {
                const uint32_t lp = ax.unc[i];
                exact_contrib(ax, lp / kBlk + goff, val_of(keys[lp]), M, T, e0);
            }
        }
        __syncthreads();
        if (!leader) {// ship the helper's block sums to the leader
            for (uint32_t i = tid; i < my_nblk; i += kThreads) {
                const uint32_t g = i + goff;
#pragma unroll
                for (int d = 0; d < kLevels; ++d) peer_ax->C[d][g] = ax.C[d][g];
                peer_ax->tie[g] = ax.tie[g];
            }
        }
        cluster.sync();// CS6
        if (leader && warp == 0) {
            uint32_t m = (__float_as_uint(s_base) & 0x7FFFFFu) | 0x800000u;
            int level = 0;
            bool again = false;
            float s_cur = s_base;
            uint32_t b0 = gb_first;
            while (b0 < nblk) {
                const uint32_t b = b0 + lane;
                const uint32_t raw = b < nblk ? ax.C[level][b] : 0u;
                const bool tied = b < nblk && ((ax.tie[b] >> level) & 1u);
                uint32_t inc = min(raw, 1u << 25);// >= 2^24 is a carry by itself; keeps the scan in 32 bits
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += t;
                }
                const uint32_t evm = __ballot_sync(0xffffffffu, tied || (m + inc >= (1u << 24)));
                if (evm == 0) {
                    m += __shfl_sync(0xffffffffu, inc, 31);
                    b0 += 32;
                    continue;
                }
                const int l = __ffs(evm) - 1;
                m += l == 0 ? 0u : __shfl_sync(0xffffffffu, inc, l - 1);
                const uint32_t eb = b0 + l;// replay this block with real fp32 additions
                float s_new = __uint_as_float((uint32_t) (e0 + level - 23) << 23) * (float) m;
                {
                    const uint16_t *blk = eb < nblk0 ? keys + eb * kBlk : peer_keys + (eb - nblk0) * kBlk;
                    const uint32_t gbase = eb < nblk0 ? eb * kBlk : (uint32_t) kHalfElems + (eb - nblk0) * kBlk;
                    uint32_t kk[8];
                    lds_keys(blk + lane * 8, kk);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const uint32_t j = gbase + lane * 8 + e;
                        ax.blk_terms[lane * 8 + e] = (kk[e] == 0 || j < pos) ? 0.f : term_of(val_of(kk[e]), M, T);
                    }
                    __syncwarp();
                    if (lane == 0) {
                        for (int i = 0; i < kBlk; ++i) s_new = __fadd_rn(s_new, ax.blk_terms[i]);
                    }
                    s_new = __shfl_sync(0xffffffffu, s_new, 0);
                }
                s_cur = s_new;
                const int es = (int) ((__float_as_uint(s_new) >> 23) & 0xFFu);
                level = es - e0;
                m = (__float_as_uint(s_new) & 0x7FFFFFu) | 0x800000u;
                b0 = eb + 1;
                if (level >= kLevels) {
                    again = b0 < nblk;
                    break;
                }
            }
            if (b0 >= nblk && level < kLevels) {
                s_cur = __uint_as_float((uint32_t) (e0 + level - 23) << 23) * (float) m;
            }
            if (lane == 0) {
                ax.mail.s_base = s_cur;
                ax.mail.pos_base = b0 * kBlk;
                ax.mail.done = again ? 0 : 1;
                peer_ax->mail.s_base = s_cur;
                peer_ax->mail.pos_base = b0 * kBlk;
                peer_ax->mail.done = again ? 0 : 1;
            }
        }
        cluster.sync();// CS7
    }
    stamp();// 5: denominator

    // ---- probabilities of the top-k, top-p cut, pick -------------------------------------
    if (leader && warp == 0) {
        const float S = ax.mail.s_base;
        for (int i = lane; i < k; i += 32) ax.top_term[i] = f16_to_f32(f32_to_f16_ref(__fdiv_rn(ax.top_term[i], S)));
        __syncwarp();
        if (lane == 0) {
            if (a.debug) {
                float *dbg = a.debug + (int64_t) row * kDebugStride;
                dbg[0] = S;
                for (int i = 0; i < k && i < kSlots; ++i) {
                    dbg[1 + i] = __uint_as_float(ax.top_idx[i]);
                    dbg[1 + kSlots + i] = ax.top_term[i];
                }
                dbg[129 + 15] = (float) rounds;
            }
            pick_from_topk(ax.top_term, ax.top_idx, k, a.topp, random_val, a.result + (int64_t) row * a.result_stride);
        }
    }
}

}// namespace

namespace b200 {

// Sampling branch for rows of at most 131072 logits and topk <= 64.
bool random_sample_pair_supported(int voc) { return voc >= 1 && voc <= 2 * kHalfElems; }

infiniopStatus_t random_sample_pair_launch(const RandomSampleArgs &a, int rows, cudaStream_t st) {
    static thread_local int configured_dev = -1;
    int dev = -1;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        if (cudaFuncSetAttribute(random_sample_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int) kSmemBytes) != cudaSuccess) {
            cudaGetLastError();
            return STATUS_EXECUTION_FAILED;
        }
        configured_dev = dev;
    }
    random_sample_pair_kernel<<<2 * rows, kThreads, kSmemBytes, st>>>(a);
    return check_launch("random_sample_pair");
}

}// namespace b200
