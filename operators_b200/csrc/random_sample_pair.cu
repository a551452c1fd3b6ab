// Random sample, shared-memory resident form: a thread-block cluster of two
// CTAs owns one row of up to 131072 logits, a cluster of four a row of up to
// 262144 (the cluster size is a launch attribute; the kernel reads it).
//
// Same result as random_sample_kernel (random_sample.cu), i.e. the index the
// reference CPU backend returns (src/ops/random_sample/cpu/random_sample.cc:
// 45-129); see that file's header for the three facts the algorithm rests on
// (streaming insertion, closed form of the permuted row, binade-wise integer
// sum).  What differs is where the row lives and how the work is spread:
//
//  * The row is read from HBM exactly once and kept in shared memory as the
//    fp16 bit patterns it came as: CTA r holds elements [65536 r, 65536 (r + 1));
//    CTA 0 leads, the others help.  Every later step runs on shared memory; the two CTAs
//    exchange lists, thresholds and block sums through distributed shared
//    memory and meet at hardware cluster barriers (no flag spinning anywhere).
//  * The serial parts are cut into pieces that run side by side.  The record
//    chain is split into segments that end at 128, 256, ..., 65536 (and the
//    helper half); the k largest keys at each boundary come from a selection
//    over about 2k values (lower bounds from maxima of thread groups decide
//    which values), one warp per boundary; one ordered list per half, built by
//    a single scan, feeds the top-k candidates, those selections and the records.
//  * The denominator is formed for FOUR binades of the running sum at once:
//    per element z = 2*term/ulp0 comes from the special-function unit
//    (ex2.approx), floor(z) gives round-to-nearest(term/ulp_d) for d = 0..3 with
//    shifts, and only elements whose z lies within the approximation's error
//    band of an integer (or that are very large) are re-evaluated exactly with
//    a double-precision exp, densely, by the whole CTA.  The walk over the
//    256-element block sums looks at all of them at once and replays, with real
//    fp32 additions, each block in which the running sum may change binade.
#include "common.cuh"
#include "random_sample.cuh"
#include "random_sample_device.cuh"

#include <cooperative_groups.h>
#include <cstddef>

namespace cg = cooperative_groups;
using namespace b200;

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kBlk = 256;
constexpr int kFlatCap = 1024;    // per-CTA ordered list (candidates, flagged records)
constexpr int kHalfElems = 65536; // elements held by one CTA
constexpr int kMaxRanks = 4;       // CTAs per cluster: 2 up to 131072 logits, 4 up to 262144
constexpr int kMaxBlk = kMaxRanks * kHalfElems / kBlk;
constexpr int kLevels = 4;
constexpr int kUncCap = 6144;
constexpr int kMaxRounds = 6;     // 6 x 4 binades covers any sum of <= 2^18 terms <= 1 (18 binades above 1)
constexpr int kTieGroups = 64;
// Record segments of the leader's part end at these positions (each twice the one before, so every
// segment holds about k flagged entries and 0.7 k records whatever its length); every helper's part
// is one more segment.  The k largest keys of a prefix that ends at one of the first kDirect boundaries
// are found directly on the row; for the later boundaries they come from a candidate list whose
// threshold is a lower bound taken from maxima of groups of threads.  Those prefixes are covered by
// whole per-thread load slots: thread t's vector u is elements [8t + 8192u, 8t + 8192u + 8).
constexpr int kWalkWarps = kMaxBlk / 32;// the walk looks at all block sums at once, 32 per warp
constexpr int kBounds = 10;
constexpr int kDirect = 2;
__device__ __constant__ uint32_t kBoundPos[kBounds] = {128u, 256u, 512u, 1024u, 2048u, 4096u, 8192u, 16384u, 32768u, 65536u};
// Scan assignment of the leader's part: warp w looks at [kScanR0[w], kScanR0[w + 1]), which lies inside
// segment kScanSeg[w].  Pieces shorter than 256 are cut into 64-element chunks, the others into
// 256-element blocks (at most 16 per warp).
__device__ __constant__ uint32_t kScanR0[kWarps + 1] = {
    0u, 64u, 128u, 192u, 256u, 384u, 512u, 768u, 1024u, 1536u, 2048u, 3072u, 4096u, 6144u, 8192u, 12288u,
    16384u, 20480u, 24576u, 28672u, 32768u, 36864u, 40960u, 45056u, 49152u, 53248u, 57344u, 61440u, 65536u,
    65536u, 65536u, 65536u, 65536u};
__device__ __constant__ uint8_t kScanSeg[kWarps] = {0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7,
                                                    8, 8, 8, 8, 9, 9, 9, 9, 9, 9, 9, 9, 9, 9, 9, 9};
constexpr uint32_t kEmptyMin = 0xFFFFFFFFu;
constexpr uint16_t kPad = 0xFC00u;// fp16 -inf: never a candidate, contributes nothing

// Ordered (index order) list of (position, key) pairs.  Slots [0, kFlatCap) hold
// this CTA's entries; at the leader, slots [kFlatCap, 2*kFlatCap) receive the
// helper's entries.
struct FlatList {
    uint32_t idx[2 * kFlatCap];
    uint16_t key[2 * kFlatCap];
    int cnt;      // own entries
    int overflow; // own entries did not fit
    int peer_cnt[kMaxRanks - 1];// leader: entries of helper 1, 2, 3 (each in its own share of the upper slots)
    int peer_overflow;
    int wcnt[kWarps];          // entries found by each warp of the scan
    int seg_first[kBounds + 1];// leader: list position of the first entry of segment i; [kBounds] = count
};
// Records to replay: the entries of the ordered list that lie above the k-th largest key at the start
// of their segment, in index order.
struct RecList {
    uint32_t idx[kFlatCap];
    uint16_t key[kFlatCap];
    int cnt;
    int seg_first[kBounds + 1];// leader: position of the first entry of segment i; [kBounds] = count
};
struct Mail {// written by other CTAs of the cluster (the leader also fills its own copy)
    uint32_t L_of[kMaxRanks];// every CTA's lower bound of the k-th largest key of its own part
    uint32_t mkey;
    float s_base;
    uint32_t pos_base;
    int done;
};
struct Aux {
    FlatList fl;
    RecList rl;
    alignas(16) uint16_t gbuf[2 * kFlatCap];// start states: 256 fp16 values per boundary; then top-k: per-key-group queues of candidate ordinals
    int state_ovf;                         // a boundary had more than 256 values to choose from
    int wcnt_r[kWarps], wcnt_h[kWarps];    // per-warp counts of the list compaction (records, helper's candidates)
    uint32_t tie_key[kTieGroups];
    uint32_t tie_greater[kTieGroups];
    uint32_t tie_same[kTieGroups];
    int tie_groups;
    uint32_t top_key[kSlots];
    uint32_t top_idx[kSlots];
    alignas(16) float top_term[kSlots];
    alignas(16) float blk_terms[kBlk];
    uint32_t walk_event;                   // block to replay with real additions, or none
    uint32_t walk_tot[kWalkWarps], walk_m[kWalkWarps];
    int walk_ev[kWalkWarps];
    float walk_s;
    uint32_t tie_excl[kBlk], tie_c[kBlk];  // integer replay of a block: prefix and own contribution per element
    uint32_t C[kLevels][kMaxBlk];// integer block sums per binade level
    uint32_t tie[kMaxBlk];       // bit d: block holds an exact half-way case at level d
    uint32_t LB[kBounds];        // lower bound of the k-th largest key of the prefix that ends at boundary b
    uint32_t seg_tau[kBounds + 1];       // exact k-th largest key at the start of segment i
    uint32_t state[kBounds + 1][kSlots]; // the k largest keys at the start of segment i (slot order irrelevant)
    alignas(16) uint32_t unc[kUncCap];// positions (local) to re-evaluate exactly; before that, the per-thread maxima (read as 16-byte vectors)
    int unc_cnt;
    Mail mail;
};

constexpr size_t kSmemBytes = (size_t) kHalfElems * 2 + sizeof(Aux);
static_assert(offsetof(Aux, unc) % 16 == 0 && (kHalfElems * 2) % 16 == 0, "vector loads from the maxima arrays");
static_assert(kSmemBytes <= 227 * 1024, "row half + bookkeeping must fit one SM's shared memory");

__device__ __forceinline__ uint16_t half_of_key(uint32_t key) {
    return key >= 0x8000u ? (uint16_t) (key - 0x8000u) : (uint16_t) (0x8000u | (0x8000u - key));
}
__device__ __forceinline__ __half2 h2_of(uint32_t w) { return *reinterpret_cast<const __half2 *>(&w); }

// 8 consecutive fp16 values (4 packed words) against a threshold: bit e of the
// result is set when element e is > thr (strict) or >= thr.
__device__ __forceinline__ uint32_t flag8(const uint32_t w[4], __half2 thr2, bool strict) {
    uint32_t m[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) m[q] = strict ? __hgt2_mask(h2_of(w[q]), thr2) : __hge2_mask(h2_of(w[q]), thr2);
    // element 2q -> bit 2q, element 2q+1 -> bit 16 + 2q + 1, then fold the upper half down
    const uint32_t p = (m[0] & 0x00020001u) | (m[1] & 0x00080004u) | (m[2] & 0x00200010u) | (m[3] & 0x00800040u);
    return (p | (p >> 16)) & 0xFFu;
}
__device__ __forceinline__ void lds_raw(const uint16_t *p, uint32_t w[4]) {
    const uint4 v = *reinterpret_cast<const uint4 *>(p);
    w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
}
__device__ __forceinline__ uint16_t half_at(const uint32_t *w, int e) { return (uint16_t) (w[e >> 1] >> ((e & 1) * 16)); }
__device__ __forceinline__ __half2 thr2_of_key(uint32_t key) {
    // keys below 0x0400 lie under every fp16 value (0x0400 is -inf): compare with -inf then
    const uint32_t th = key < 0x0400u ? kPad : half_of_key(key);
    return h2_of(th | (th << 16));
}

// One warp holds n_vec8 * 8 fp16 values (shared memory at p, 16-byte aligned) in registers, NW packed
// words per lane (NW * 64 >= n_vec8 * 8; missing ones are -inf), and bisects on them without touching
// memory again.
template<int NW>
struct WarpVals {
    uint32_t w[NW];
    __device__ __forceinline__ void load(const uint16_t *p, int n_vec8, int lane) {
#pragma unroll
        for (int j = 0; j < NW / 4; ++j) {
            const int v = lane + 32 * j;
            uint4 q = make_uint4(0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u);
            if (v < n_vec8) q = *reinterpret_cast<const uint4 *>(p + v * 8);
            w[4 * j] = q.x, w[4 * j + 1] = q.y, w[4 * j + 2] = q.z, w[4 * j + 3] = q.w;
        }
    }
    // this lane's count of values >= thr (or > thr)
    __device__ __forceinline__ int count(__half2 thr2, bool strict) const {
        int c = 0;
#pragma unroll
        for (int g = 0; g < NW; g += 16) {
            uint32_t acc = 0;// word r of the group answers in bits r and 16 + r
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                if (g + r < NW) {
                    const uint32_t m = strict ? __hgt2_mask(h2_of(w[g + r]), thr2) : __hge2_mask(h2_of(w[g + r]), thr2);
                    acc |= m & (0x00010001u << r);
                }
            }
            c += __popc(acc);
        }
        return c;
    }
    // this lane's counts of values >= each of three thresholds, in the low and high half of x and in y
    __device__ __forceinline__ void count3(__half2 t1, __half2 t2, __half2 t3, uint32_t &x, uint32_t &y) const {
        uint32_t c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
        for (int g = 0; g < NW; g += 16) {
            uint32_t a1 = 0, a2 = 0, a3 = 0;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                if (g + r < NW) {
                    const uint32_t sel = 0x00010001u << r;
                    a1 |= __hge2_mask(h2_of(w[g + r]), t1) & sel;
                    a2 |= __hge2_mask(h2_of(w[g + r]), t2) & sel;
                    a3 |= __hge2_mask(h2_of(w[g + r]), t3) & sel;
                }
            }
            c1 += __popc(a1), c2 += __popc(a2), c3 += __popc(a3);
        }
        x = c1 | (c2 << 16);
        y = c3;
    }
    // Key of the k-th largest value (with multiplicity); 0x0400 (the key of -inf) when fewer than k
    // values lie above -inf.  Four-way search: three thresholds per step, eight steps.
    __device__ __forceinline__ uint32_t kth_largest(int k, uint32_t lo_hint) const {
        // the search runs between the smallest value (or a bound the caller knows to have k values at or
        // above it) and the largest one: a few hundred to a few thousand keys instead of all 63488
        __half2 mn2 = h2_of(w[0]), mx2 = mn2;
#pragma unroll
        for (int r = 1; r < NW; ++r) {
            mn2 = __hmin2(mn2, h2_of(w[r]));
            mx2 = __hmax2(mx2, h2_of(w[r]));
        }
        const uint32_t kmin = key_of(__half_as_ushort(__hmin(__low2half(mn2), __high2half(mn2))));
        const uint32_t kmax = key_of(__half_as_ushort(__hmax(__low2half(mx2), __high2half(mx2))));
        uint32_t lo = max(max(__reduce_min_sync(0xffffffffu, kmin), lo_hint), 0x0400u);
        uint32_t hi = max(__reduce_max_sync(0xffffffffu, kmax), lo);
        while (lo < hi) {
            const uint32_t m2 = (lo + hi + 1) >> 1;// lo < m2 <= hi
            const uint32_t m1 = (lo + m2) >> 1;    // lo <= m1 < m2
            const uint32_t m3 = (m2 + hi + 1) >> 1;// m2 <= m3 <= hi
            uint32_t x, y;
            count3(thr2_of_key(m1), thr2_of_key(m2), thr2_of_key(m3), x, y);
            x = __reduce_add_sync(0xffffffffu, x);// at most 2048 values: the halves do not carry
            y = __reduce_add_sync(0xffffffffu, y);
            const int c1 = (int) (x & 0xFFFFu), c2 = (int) (x >> 16), c3 = (int) y;
            if (c3 >= k) lo = m3;
            else if (c2 >= k) lo = m2, hi = m3 - 1;
            else if (c1 >= k) lo = m1, hi = m2 - 1;
            else hi = m1 - 1;// below lo when m1 == lo: ends the search with lo unchanged
        }
        return lo;
    }
    // The k largest keys into st[0, k): those above tau (fewer than k), then copies of tau.
    __device__ __forceinline__ void k_largest(uint32_t tau, int k, uint32_t *st, int lane) const {
        const __half2 t2 = thr2_of_key(tau);
        const int mine = count(t2, true);
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        int at = incl - mine;
#pragma unroll
        for (int r = 0; r < NW; ++r) {
            const uint32_t m = __hgt2_mask(h2_of(w[r]), t2);
            if (m & 0xFFFFu) st[at++] = key_of((uint16_t) (w[r] & 0xFFFFu));
            if (m >> 16) st[at++] = key_of((uint16_t) (w[r] >> 16));
        }
        const int filled = __shfl_sync(0xffffffffu, incl, 31);
        for (int sl = filled + lane; sl < k; sl += 32) st[sl] = tau;
    }
};

// Key of the k-th largest of up to 256 fp16 values (n_vec8 vectors of 8 at p); with st, also the k
// largest keys into st[0, k).  lo_hint: a key known to have at least k values at or above it (or 0).  One warp; one copy of the code for all the warps that call it.
__device__ __noinline__ uint32_t kth_largest_256(const uint16_t *p, int n_vec8, int k, uint32_t *st, uint32_t lo_hint) {
    const int lane = threadIdx.x & 31;
    WarpVals<4> v;
    v.load(p, n_vec8, lane);
    const uint32_t tau = v.kth_largest(k, lo_hint);
    if (st != nullptr) v.k_largest(tau, k, st, lane);
    return tau;
}

// Running multiset of the k largest keys seen so far, 2 slots per lane.  Each
// slot holds (key << 6) | slot_id, so that a single warp-wide minimum `p`
// returns both the k-th largest key (p >> 6) and the slot that holds it
// (p & 63).  Slots >= k hold 0xFFFFFFFF.  Because slot ids fill the low bits,
// "key > tau" is the same as "(key << 6) > p".
struct MinBuf {
    uint32_t v0, v1;// packed slots lane and lane + 32
    uint32_t p;     // packed minimum
    __device__ __forceinline__ uint32_t tau() const { return p >> 6; }
};
__device__ __forceinline__ void minbuf_init(MinBuf &m, int lane, int k, const uint16_t *first_raw) {
    m.v0 = lane < k ? (key_of(first_raw[lane]) << 6) | (uint32_t) lane : kEmptyMin;
    m.v1 = lane + 32 < k ? (key_of(first_raw[lane + 32]) << 6) | (uint32_t) (lane + 32) : kEmptyMin;
    m.p = __reduce_min_sync(0xffffffffu, min(m.v0, m.v1));
}
__device__ __forceinline__ void minbuf_init_keys(MinBuf &m, int lane, int k, const uint32_t *keys) {
    m.v0 = lane < k ? (keys[lane] << 6) | (uint32_t) lane : kEmptyMin;
    m.v1 = lane + 32 < k ? (keys[lane + 32] << 6) | (uint32_t) (lane + 32) : kEmptyMin;
    m.p = __reduce_min_sync(0xffffffffu, min(m.v0, m.v1));
}
// Replace the smallest held key by the key in `key_shl6` (= key << 6, known to
// every lane).  The dependent chain from the old minimum to the new one is:
// mask, compare, move, min, warp-wide min.
__device__ __forceinline__ void minbuf_replace(MinBuf &m, int lane, uint32_t key_shl6) {
    const uint32_t slot = m.p & 63u;
    const uint32_t np = key_shl6 | slot;
    if ((uint32_t) lane == slot) m.v0 = np;
    if ((uint32_t) lane + 32u == slot) m.v1 = np;
    m.p = __reduce_min_sync(0xffffffffu, min(m.v0, m.v1));
}

// One warp walks a 256-element block (local or the peer's shared memory) in
// index order and feeds every element above the running k-th largest value;
// a record is overwritten with that value.  Slow path (list overflow only).
__device__ __noinline__ void records_direct_block(uint16_t *blk, uint32_t first_in_blk, int lane, MinBuf &m) {
    uint32_t w[4], keys[8];
    lds_raw(blk + lane * 8, w);
#pragma unroll
    for (int e = 0; e < 8; ++e) keys[e] = half_at(w, e) == kPad ? 0u : key_of(half_at(w, e));
    uint32_t mask = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        if ((uint32_t) (lane * 8 + e) >= first_in_blk && keys[e] > m.tau()) mask |= 1u << e;
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
        if (lane == src) mask &= mask - 1;
        if (key > m.tau()) {
            if (lane == 0) blk[src * 8 + e] = half_of_key(m.tau());
            minbuf_replace(m, lane, key << 6);
            // the bar moved: drop what no longer clears it
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                if (keys[t] <= m.tau()) mask &= ~(1u << t);
            }
        }
        any = __ballot_sync(0xffffffffu, mask != 0);
    }
}

// Warp 0 replays an ordered list of (position, key): every entry above the
// running k-th largest value is a record and is overwritten with that value in
// `dst` (positions are taken relative to `pos_offset`).  Sixteen keys at a time
// are read into registers of every lane, so the only serial dependency between
// entries is the running value itself (one warp-wide minimum per record).
__device__ __noinline__ void replay_list(const uint16_t *keys, const uint32_t *idx, int count, uint16_t *dst,
                                         uint32_t pos_offset, int lane, MinBuf &m) {
    constexpr int kBatch = 16;
    for (int c0 = 0; c0 < count; c0 += kBatch) {
        uint32_t kb[kBatch];// key << 6
#pragma unroll
        for (int i = 0; i < kBatch; ++i) kb[i] = c0 + i < count ? (uint32_t) keys[c0 + i] << 6 : 0u;
        const uint32_t my_idx = (lane < kBatch && c0 + lane < count) ? idx[c0 + lane] : 0u;
        uint32_t my_tau = kEmptyMin;// lane i remembers the value its entry is replaced by; stored after the batch
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            if (kb[i] > m.p) {// key > tau, uniform across the warp
                if (lane == i) my_tau = m.tau();
                minbuf_replace(m, lane, kb[i]);
            }
        }
        if (my_tau != kEmptyMin) dst[my_idx - pos_offset] = half_of_key(my_tau);
    }
}

// exp in double precision is some hundred instructions: one copy, called.
__device__ __noinline__ float term_exact(float v, float M, float T) { return term_of(v, M, T); }

// Exact contribution of one term to the block sums of all levels.
__device__ __noinline__ void exact_contrib(Aux &ax, uint32_t blk, float v, float M, float T, int e0) {
    const uint32_t tb = __float_as_uint(term_exact(v, M, T));
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

// The same split for one level: what the term adds to the mantissa of a running sum whose ulp is
// 2^(e0 + level - 150), and whether it lies exactly half-way (then the addition rounds to even).
__device__ __forceinline__ void exact_at_level(float term, int e0, int level, uint32_t &c, bool &tie) {
    const uint32_t tb = __float_as_uint(term);
    int e_t = (int) ((tb >> 23) & 0xFFu);
    uint32_t man = tb & 0x7FFFFFu;
    if (e_t == 0) e_t = 1;
    else man |= 0x800000u;
    const int sh = e0 + level - e_t;
    c = 0, tie = false;
    if (man == 0 || sh >= 25) return;
    const uint32_t rem = man & ((1u << sh) - 1u);
    const uint32_t half = sh > 0 ? 1u << (sh - 1) : 0u;
    c = (man >> sh) + ((sh > 0 && rem > half) ? 1u : 0u);
    tie = sh > 0 && rem == half;
}

// ---- peer memory (vocabulary-sharded rows) ----------------------------------------------
constexpr long long kPeerWaitBudget = 2000ll * 1000 * 1000;// clock64 ticks, about a second
__device__ unsigned long long g_pair_peer_timeouts = 0;

__device__ __forceinline__ void peer_st_release(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void peer_st_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint4 peer_ld_v4(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// Until *flag has reached `call` (the counters wrap; the difference counts).  Bounded: a wait that runs out is counted.
__device__ __forceinline__ void peer_wait(const uint32_t *flag, uint32_t call) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int32_t) (v - call) >= 0) return;
        if (clock64() - t0 > kPeerWaitBudget) {
            atomicAdd(&g_pair_peer_timeouts, 1ull);
            return;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1) random_sample_pair_kernel(RandomSampleArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint16_t *raw = reinterpret_cast<uint16_t *>(smem_raw);// this CTA's part of the row, fp16 bit patterns
    Aux &ax = *reinterpret_cast<Aux *>(smem_raw + (size_t) kHalfElems * 2);
    cg::cluster_group cluster = cg::this_cluster();
    // CTA `rank` of the cluster holds elements [rank * 65536, (rank + 1) * 65536) of the row; rank 0 leads.
    const unsigned rank = cluster.block_rank(), R = cluster.num_blocks();
    const bool leader = rank == 0;
    // the same objects in another CTA of the cluster (one address-mapping instruction each time)
    auto ax_of = [&](unsigned r) -> Aux * { return cluster.map_shared_rank(&ax, r); };
    Aux *lead_ax = ax_of(0);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x / R;
    const uint32_t n = (uint32_t) a.voc;
    const uint32_t n0 = min(n, (uint32_t) kHalfElems);// leader's elements
    const uint32_t my_base = rank * (uint32_t) kHalfElems;
    const uint32_t my_n = n > my_base ? min(n - my_base, (uint32_t) kHalfElems) : 0u;
    const uint32_t my_nblk = (my_n + kBlk - 1) / kBlk;
    const uint32_t my_pad = my_nblk * kBlk;
    const uint32_t nblk0 = (n0 + kBlk - 1) / kBlk;
    const uint32_t nblk = (n + kBlk - 1) / kBlk;// every part before the last is full: block g lives in CTA g / 256
    const uint32_t ranks_used = (n + kHalfElems - 1) / kHalfElems;// CTAs that hold data
    const uint16_t *logits = a.logits + (int64_t) row * a.logits_stride + my_base;
    const float random_val = a.random_vals ? a.random_vals[row] : a.random_val;
    const float T = a.temperature;
    const int k = a.topk > (int) n ? (int) n : a.topk;

    const long long t_entry = clock64();
    int stamp_i = 0;
    auto stamp = [&]() {
        if (a.debug && leader && tid == 0 && stamp_i < 6) {
            a.debug[(int64_t) row * kDebugStride + 129 + stamp_i] = (float) (clock64() - t_entry);
        }
        ++stamp_i;
    };

    auto block_ptr = [&](uint32_t g) -> const uint16_t * {
        return cluster.map_shared_rank(raw, g >> 8) + (g & 255u) * kBlk;
    };

    // ---- sharded rows: tell the peers that this rank's shard is final, wait for theirs ----
    const PeerRowSource &pr = a.peer;
    uint32_t peer_call = 0;
    if (pr.world) {
        uint32_t *mine = pr.flags[pr.rank];
        peer_call = mine[kPeerCalls] + 1;// raised by the CTA that finishes last, after every CTA has read it
        if (blockIdx.x == 0 && tid < (int) pr.world) peer_st_release(&pr.flags[tid][kPeerReady + pr.rank], peer_call);
        if (tid < (int) pr.world && tid != (int) pr.rank) peer_wait(&mine[kPeerReady + tid], peer_call);
        __syncthreads();// a wait that ran out is counted; the row is then sampled from what the shard holds
    }
    // vector v (8 elements) of this CTA's part of the row
    auto vec_src = [&](uint32_t base) -> const uint16_t * {
        if (!pr.world) return logits + base;
        const uint32_t gv = (my_base + base) >> 3, p = gv / pr.shard_vecs;
        return pr.shard[p] + (int64_t) (pr.row0 + row) * pr.shard_stride[p] + (size_t) (gv - p * pr.shard_vecs) * 8;
    };

    // ---- P1: this CTA's part of the row -> shared memory; per-thread maxima --------------
    const bool in_aligned = pr.world != 0 || (reinterpret_cast<uintptr_t>(logits) & 15u) == 0;
    __half2 tmax2 = h2_of(0xFC00FC00u), m0_2 = tmax2, mA_2 = tmax2, mB_2 = tmax2;// running maximum; after 1, 2 and 4 vectors
    auto max4 = [](const uint4 q) { return __hmax2(__hmax2(h2_of(q.x), h2_of(q.y)), __hmax2(h2_of(q.z), h2_of(q.w))); };
    constexpr int kInFlight = 8;
    for (uint32_t base0 = tid * 8; base0 < my_pad; base0 += kThreads * 8 * kInFlight) {// whole aligned vectors
        uint4 ld[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t base = base0 + u * kThreads * 8;
            ld[u] = make_uint4(0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u);
            // peer memory: volatile, so that no line of an earlier call's logits comes out of L1
            if (in_aligned && base + 8 <= my_n) ld[u] = pr.world ? peer_ld_v4(vec_src(base)) : ld_stream(logits + base);
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t base = base0 + u * kThreads * 8;
            if (base < my_pad) {
                *reinterpret_cast<uint4 *>(raw + base) = ld[u];
                tmax2 = __hmax2(tmax2, max4(ld[u]));
            }
            if (u == 0) m0_2 = tmax2;
            if (u == 1) mA_2 = tmax2;
            if (u == 3) mB_2 = tmax2;
        }
    }
    if (!in_aligned || (my_n & 7u)) {// ragged end or unaligned row: those vectors again, element-wise, padded with -inf
#pragma unroll 1
        for (uint32_t base = tid * 8; base < my_pad; base += kThreads * 8) {
            if (in_aligned && base + 8 <= my_n) continue;
            uint16_t h[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) h[e] = base + e < my_n ? logits[base + e] : kPad;
            const uint4 q = make_uint4(h[0] | ((uint32_t) h[1] << 16), h[2] | ((uint32_t) h[3] << 16),
                                       h[4] | ((uint32_t) h[5] << 16), h[6] | ((uint32_t) h[7] << 16));
            *reinterpret_cast<uint4 *>(raw + base) = q;
            const __half2 vm = max4(q);
            const uint32_t u = base / (kThreads * 8);
            tmax2 = __hmax2(tmax2, vm);
            if (u == 0) m0_2 = __hmax2(m0_2, vm);
            if (u <= 1) mA_2 = __hmax2(mA_2, vm);
            if (u <= 3) mB_2 = __hmax2(mB_2, vm);
        }
    }
    // Maxima of disjoint groups of elements (fp16; -inf = nothing but padding), at most 256 per
    // boundary from 512 on: x_b[g] is the maximum of the part of group g that lies below boundary b
    // (a group is one thread's slots, or two or four neighbouring threads').  The k-th largest entry
    // of x_b is a lower bound of the k-th largest key of that prefix, because k different elements
    // of the prefix are at least that large.  One warp per boundary finds it; two more warps find
    // the exact k largest keys of the prefixes 128 and 256 on the row itself.
    // state b + 1 (the k largest keys of the prefix that ends at boundary b) is wanted when a segment starts there
    auto need_state = [&](int b) { return kBoundPos[b] < n0 || (kBoundPos[b] == n0 && n > n0); };
    {
        uint16_t *xs = reinterpret_cast<uint16_t *>(ax.unc);// [kBounds - kDirect][256], free until the denominator
        auto one = [](const __half2 m2) { return __hmax(__low2half(m2), __high2half(m2)); };
        const __half x0 = one(m0_2);
        __half2 p01 = __halves2half2(x0, one(mA_2)), p23 = __halves2half2(one(mB_2), one(tmax2));
        const __half2 q01 = __hmax2(p01, __shfl_xor_sync(0xffffffffu, p01, 1));
        p01 = __hmax2(q01, __shfl_xor_sync(0xffffffffu, q01, 2));// maxima over four neighbouring threads
        p23 = __hmax2(p23, __shfl_xor_sync(0xffffffffu, p23, 1));
        p23 = __hmax2(p23, __shfl_xor_sync(0xffffffffu, p23, 2));
        if (tid < 64) xs[0 * 256 + tid] = __half_as_ushort(x0); // below 512
        if (tid < 128) xs[1 * 256 + tid] = __half_as_ushort(x0);// below 1024
        if (tid < 256) xs[2 * 256 + tid] = __half_as_ushort(x0);// below 2048
        if (tid < 512 && !(tid & 1)) xs[3 * 256 + (tid >> 1)] = __half_as_ushort(__low2half(q01));// below 4096
        if (!(tid & 3)) {
            xs[4 * 256 + (tid >> 2)] = __half_as_ushort(__low2half(p01)); // below 8192
            xs[5 * 256 + (tid >> 2)] = __half_as_ushort(__high2half(p01));// below 16384
            xs[6 * 256 + (tid >> 2)] = __half_as_ushort(__low2half(p23)); // below 32768
            xs[7 * 256 + (tid >> 2)] = __half_as_ushort(__high2half(p23));// all
        }
        __syncthreads();
        if (warp < kBounds - kDirect && (leader || warp == kBounds - kDirect - 1)) {
            const uint32_t kth = kth_largest_256(xs + warp * 256, warp == 0 ? 8 : warp == 1 ? 16 : 32, k, nullptr, 0u);
            if (lane == 0) ax.LB[kDirect + warp] = kth <= 0x0400u ? 1u : kth;// fewer than k groups hold data: everything
        } else if (leader && warp >= kBounds - kDirect && warp < kBounds && (uint32_t) k < n &&
                   need_state(warp - (kBounds - kDirect))) {
            const int b = warp - (kBounds - kDirect);
            const uint32_t tau = kth_largest_256(raw, (int) (kBoundPos[b] / 8u), k, ax.state[b + 1], 0u);
            if (lane == 0) ax.seg_tau[b + 1] = tau;
        } else if (leader && warp == kBounds && (uint32_t) k < n) {// the k-th largest of the first k elements
            MinBuf fb;
            minbuf_init(fb, lane, k, raw);
            if (lane == 0) ax.seg_tau[0] = fb.tau();
        }
        __syncthreads();
    }
    const uint32_t L_mine = ax.LB[kBounds - 1];
    if (tid < (int) R) ax_of((unsigned) tid)->mail.L_of[rank] = my_n > 0 ? L_mine : 0u;
    if (tid == 0) {
        ax.state_ovf = 0;
        for (int h = 0; h < kMaxRanks - 1; ++h) ax.fl.peer_cnt[h] = 0;// the helpers fill these in after the barrier
        ax.fl.peer_overflow = 0;
    }
    cluster.sync();// CS1
    stamp();       // 0: row resident
    uint32_t L = 1u, L_before = 0u;// L_before: a lower bound of the k-th largest key of everything before this part
    for (unsigned r = 0; r < R; ++r) {
        L = max(L, ax.mail.L_of[r]);
        if (r < rank) L_before = max(L_before, ax.mail.L_of[r]);
    }

    // ---- P2: candidates (key >= L), ordered --------------------------------------------
    // Ordered list of the elements of this warp's piece [r0, r1) of the LOCAL half that lie above
    // (strict) or at or above the key `tk`, positions below e_begin left out.  Two passes: every
    // warp flags its piece into registers (one byte per 256-element block or 64-element chunk) and
    // counts; after one CTA barrier each warp knows where its entries go and writes them in index
    // order.  All threads of the CTA call it; `cap` is the room in the list.
    auto scan_ordered = [&](uint32_t r0, uint32_t r1, uint32_t e_begin, uint32_t tk, bool strict, int cap) {
        const __half2 thr2 = thr2_of_key(tk);
        const bool fine = r1 - r0 < (uint32_t) kBlk;// whole pieces are multiples of 64 or of 256
        r1 = min(r1, my_n);                         // padding beyond the real end is never listed
        uint32_t pm[4] = {0u, 0u, 0u, 0u};         // flags of piece i: byte i & 3 of pm[i >> 2]
        if (r0 < r1) {
            if (fine) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const uint32_t c = r0 + 64u * i;
                    if (c < r1) {
                        const uint32_t w2 = *reinterpret_cast<const uint32_t *>(raw + c + lane * 2);
                        const uint32_t mm = strict ? __hgt2_mask(h2_of(w2), thr2) : __hge2_mask(h2_of(w2), thr2);
                        const uint32_t j = c + lane * 2;
                        uint32_t mask = 0;
                        if ((mm & 1u) && j >= e_begin && j < r1) mask |= 1u;
                        if ((mm >> 16) && j + 1 >= e_begin && j + 1 < r1) mask |= 2u;
                        pm[0] |= mask << (8 * i);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t c = r0 + (uint32_t) kBlk * i;
                    if (c < r1) {
                        uint32_t w[4];
                        lds_raw(raw + c + lane * 8, w);
                        uint32_t mask = flag8(w, thr2, strict);
                        const uint32_t first = c + lane * 8;
                        if (first + 8 > r1) mask &= first >= r1 ? 0u : (1u << (r1 - first)) - 1u;
                        if (first < e_begin) mask &= first + 8 <= e_begin ? 0u : ~((1u << (e_begin - first)) - 1u);
                        pm[i >> 2] |= mask << (8 * (i & 3));
                    }
                }
            }
        }
        const int mine = __popc(pm[0]) + __popc(pm[1]) + __popc(pm[2]) + __popc(pm[3]);
        const int wtot = __reduce_add_sync(0xffffffffu, mine);
        if (lane == 0) ax.fl.wcnt[warp] = wtot;
        __syncthreads();
        const int c_l = ax.fl.wcnt[lane];// kWarps == 32: one lane per warp
        int at = __reduce_add_sync(0xffffffffu, lane < warp ? c_l : 0);
        const int tot = __reduce_add_sync(0xffffffffu, c_l);
        const bool over = tot > cap;
        if (tid == 0) {
            ax.fl.cnt = over ? 0 : tot;
            ax.fl.overflow = over ? 1 : 0;
            ax.fl.seg_first[kBounds] = tot;
        }
        if (leader && lane == 0 && (warp == 0 || kScanSeg[warp - 1] != kScanSeg[warp])) ax.fl.seg_first[kScanSeg[warp]] = at;
        if (!over && wtot > 0) {
            uint32_t nz = 0;// pieces in which this lane flagged something
#pragma unroll
            for (int i = 0; i < 16; ++i) nz |= ((pm[i >> 2] >> (8 * (i & 3))) & 0xFFu) ? 1u << i : 0u;
            uint32_t todo = __reduce_or_sync(0xffffffffu, nz);
            const int per_lane = fine ? 2 : 8;
            while (todo) {
                const int i = __ffs(todo) - 1;
                todo &= todo - 1;
                const uint32_t word = (i >> 2) == 0 ? pm[0] : (i >> 2) == 1 ? pm[1] : (i >> 2) == 2 ? pm[2] : pm[3];
                uint32_t m = (word >> (8 * (i & 3))) & 0xFFu;
                const uint32_t pos0 = r0 + (fine ? 64u : (uint32_t) kBlk) * i + lane * per_lane;
                const uint32_t any = __ballot_sync(0xffffffffu, m != 0);
                const uint32_t multi = __ballot_sync(0xffffffffu, (m & (m - 1)) != 0);
                if (multi == 0) {// the usual case: at most one hit per lane
                    if (m) {
                        const int e = __ffs(m) - 1;
                        const int q = at + __popc(any & ((1u << lane) - 1u));
                        ax.fl.idx[q] = my_base + pos0 + e;
                        ax.fl.key[q] = (uint16_t) key_of(raw[pos0 + e]);
                    }
                    at += __popc(any);
                } else {
                    const int cnt = __popc(m);
                    int incl = cnt;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int t = __shfl_up_sync(0xffffffffu, incl, o);
                        if (lane >= o) incl += t;
                    }
                    int q = at + incl - cnt;
                    while (m) {
                        const int e = __ffs(m) - 1;
                        m &= m - 1;
                        ax.fl.idx[q] = my_base + pos0 + e;
                        ax.fl.key[q] = (uint16_t) key_of(raw[pos0 + e]);
                        ++q;
                    }
                    at += __shfl_sync(0xffffffffu, incl, 31);
                }
            }
        }
        __syncthreads();
    };
    // Helpers: hand this CTA's list to the leader.  The upper half of the leader's arrays is divided evenly
    // among the helpers, in rank (= index) order; a helper keeps its list within its share.
    const int helper_cap = kFlatCap / (int) (R > 1 ? R - 1 : 1);
    auto ship_list = [&]() {
        const int at = kFlatCap + (int) (rank - 1) * helper_cap;
        for (int i = tid; i < ax.fl.cnt; i += kThreads) {
            lead_ax->fl.idx[at + i] = ax.fl.idx[i];
            lead_ax->fl.key[at + i] = ax.fl.key[i];
        }
        if (tid == 0) {
            lead_ax->fl.peer_cnt[rank - 1] = ax.fl.cnt;
            if (ax.fl.overflow) lead_ax->fl.peer_overflow = 1;
        }
    };
    // Helper part: equal spans of whole blocks per warp (at most 8), one threshold.
    auto scan_helper = [&](uint32_t tk, bool strict) {
        const uint32_t span = ((my_nblk + kWarps - 1) / kWarps) * kBlk;
        const uint32_t r0 = min(warp * span, my_pad);
        scan_ordered(r0, min(r0 + span, my_pad), 0u, tk, strict, helper_cap);
    };

    // One ordered list per CTA serves three purposes, so a segment's threshold is the lowest of what they
    // need: the candidates for the top-k (key >= L), the keys a later start state is chosen from (at or
    // above that boundary's bound), and the records to replay (above the k-th largest key at the START of
    // the segment, known exactly for the first segments and bounded from below by that boundary's bound
    // for the later ones).  The records are filtered out of the list later instead of scanning the row again.
    const bool want_records = (uint32_t) k < n;
    if (leader) {
        const int sg = kScanSeg[warp];
        uint32_t thr = L;
        if (want_records) {
            if (sg < kDirect) thr = min(L, ax.seg_tau[sg] + 1u);
            else if (sg == kDirect) thr = min(ax.seg_tau[sg] + 1u, ax.LB[sg]);
            else thr = ax.LB[sg - 1];
        }
        scan_ordered(kScanR0[warp], kScanR0[warp + 1], 0u, thr, false, kFlatCap);
    } else {
        // the bounds of the parts before this one are lower bounds of the k-th largest key where this part starts
        scan_helper(want_records ? min(L, max(L_before, 1u)) : L, false);
        ship_list();
    }
    cluster.sync();// CS2
    stamp();       // 1: candidate lists at the leader

    // ---- P3 (leader): exact top-k, start states of its record segments -----------------
    MinBuf mb{kEmptyMin, kEmptyMin, 0};
    float M = 0.f;
    bool list_ok = false;
    if (leader) {
        const int cnt0 = ax.fl.cnt;
        const int c_h0 = ax.fl.peer_cnt[0], c_h1 = ax.fl.peer_cnt[1], c_h2 = ax.fl.peer_cnt[2];
        const int cnt1 = c_h0 + c_h1 + c_h2;// the helpers' entries, taken in rank order
        list_ok = !ax.fl.overflow && !ax.fl.peer_overflow;
        if (list_ok && (uint32_t) k < n && warp >= kDirect && warp < kBounds && need_state(warp)) {
            // Start states of the segments from 512 on, one warp per boundary: the k largest keys of
            // the prefix are among the k largest of [0, 256) (known) and those master entries of the
            // segments in between that reach this boundary's bound (about k of them).  They are put
            // side by side as fp16 values and the selection that found the bounds runs on them.
            uint16_t *sc = ax.gbuf + (warp - kDirect) * 256;
            const int e0 = ax.fl.seg_first[kDirect], e1 = ax.fl.seg_first[warp + 1];
            const uint32_t lb = max(ax.LB[warp], 1u);
            for (int i = lane; i < 256; i += 32) sc[i] = kPad;
            __syncwarp();
            if (lane < k) sc[lane] = half_of_key(ax.state[kDirect][lane]);
            if (lane + 32 < k) sc[lane + 32] = half_of_key(ax.state[kDirect][lane + 32]);
            int fill = k;
#pragma unroll 1
            for (int i0 = e0; i0 < e1; i0 += 32) {
                const int i = i0 + lane;
                const uint32_t key = i < e1 ? (uint32_t) ax.fl.key[i] : 0u;
                const uint32_t hit = __ballot_sync(0xffffffffu, key >= lb);
                const int at = fill + __popc(hit & ((1u << lane) - 1u));
                if (key >= lb && at < 256) sc[at] = half_of_key(key);
                fill += __popc(hit);
            }
            __syncwarp();
            if (fill > 256) {
                if (lane == 0) ax.state_ovf = 1;
            } else {
                const uint32_t tau = kth_largest_256(sc, 32, k, ax.state[warp + 1], lb);
                if (lane == 0) ax.seg_tau[warp + 1] = tau;
            }
        }
        __syncthreads();// the start states have been read off the master list
        if (ax.state_ovf) list_ok = false;
        if (list_ok) {
            // Out of the ordered lists: the candidates proper (key >= L; the ranking below is quadratic in
            // their number), the helpers' behind the leader's own, in place; and the records to replay
            // (key above the k-th largest at the start of the entry's segment), into their own list.  One
            // entry per thread, read before the barrier and written to its new place after it.
            uint32_t my_idx = 0, my_key = 0, mv_idx = 0, mv_key = 0;
            bool keep = false, rec = false, keep_h = false;
            if (tid < cnt0) {
                my_key = ax.fl.key[tid];
                my_idx = ax.fl.idx[tid];
                keep = my_key >= L;
                const int sg = my_idx < 128u ? 0 : 25 - __clz(my_idx);// segment i ends at 128 << i
                rec = want_records && my_idx >= (uint32_t) k && my_key > ax.seg_tau[sg];
            }
            if (tid < cnt1) {
                const int slot = tid < c_h0 ? kFlatCap + tid
                                            : tid < c_h0 + c_h1 ? kFlatCap + helper_cap + (tid - c_h0)
                                                                : kFlatCap + 2 * helper_cap + (tid - c_h0 - c_h1);
                mv_idx = ax.fl.idx[slot];
                mv_key = ax.fl.key[slot];
                keep_h = mv_key >= L;
            }
            const uint32_t hit = __ballot_sync(0xffffffffu, keep), hit_r = __ballot_sync(0xffffffffu, rec);
            const uint32_t hit_h = __ballot_sync(0xffffffffu, keep_h);
            if (lane == 0) {
                ax.fl.wcnt[warp] = __popc(hit);
                ax.wcnt_r[warp] = __popc(hit_r);
                ax.wcnt_h[warp] = __popc(hit_h);
            }
            if (tid == 0) ax.tie_groups = 0;
            if (tid < kSlots) {
                ax.top_key[tid] = 0;
                ax.top_idx[tid] = 0;
            }
            __syncthreads();
            const int c_l = ax.fl.wcnt[lane], r_l = ax.wcnt_r[lane], h_l = ax.wcnt_h[lane];
            const int off = __reduce_add_sync(0xffffffffu, lane < warp ? c_l : 0);
            const int cnt0c = __reduce_add_sync(0xffffffffu, c_l);
            const int off_r = __reduce_add_sync(0xffffffffu, lane < warp ? r_l : 0);
            const int cnt_r = __reduce_add_sync(0xffffffffu, r_l);
            const int off_h = __reduce_add_sync(0xffffffffu, lane < warp ? h_l : 0);
            const int cnt1c = __reduce_add_sync(0xffffffffu, h_l);
            const int m = cnt0c + cnt1c;
            const uint32_t below = (1u << lane) - 1u;
            if (keep) {
                const int at = off + __popc(hit & below);
                ax.fl.key[at] = (uint16_t) my_key;
                ax.fl.idx[at] = my_idx;
            }
            if (keep_h) {
                const int at = cnt0c + off_h + __popc(hit_h & below);
                ax.fl.idx[at] = mv_idx;
                ax.fl.key[at] = (uint16_t) mv_key;
            }
            const int at_r = off_r + __popc(hit_r & below);// records before this entry
            if (rec) {
                ax.rl.key[at_r] = (uint16_t) my_key;
                ax.rl.idx[at_r] = my_idx;
            }
            // where each segment's records start: the list position of the segment's first entry, translated
            for (int sg = 0; sg <= kBounds; ++sg) {
                const int p0 = ax.fl.seg_first[sg];
                if (p0 == tid && tid < cnt0) ax.rl.seg_first[sg] = at_r;
                if (p0 >= cnt0 && tid == 0) ax.rl.seg_first[sg] = cnt_r;
            }
            if (tid == 0) {
                ax.fl.cnt = cnt0c;
                ax.rl.cnt = cnt_r;
            }
            __syncthreads();
            // Rank every candidate: `greater` keys above it, `same` keys equal to it.
            // A key that occurs once simply sits behind all larger keys.  Equal keys
            // form a group that behaves like a queue under the reference's insertion
            // cascade: an arriving equal key joins at the back (while the buffer has
            // room above the smaller keys), an arriving larger key moves the front
            // element to the back, or pushes it out when nothing smaller is left to
            // evict.  Each such group is replayed over the candidates in index order
            // by one warp; its final place is behind all larger keys.
            for (int c = tid; c < m; c += kThreads) {// normally one candidate per thread, m ~ 100
                const uint32_t my_key = ax.fl.key[c];
                uint32_t greater = 0, same = 0;
                bool seen_before = false;
                for (int j = 0; j < m; ++j) {
                    const uint32_t kj = ax.fl.key[j];
                    greater += kj > my_key;
                    same += kj == my_key;
                    seen_before |= (kj == my_key) && j < c;
                }
                if (same == 1) {
                    if (greater < (uint32_t) k) {
                        ax.top_key[greater] = my_key;
                        ax.top_idx[greater] = ax.fl.idx[c];
                    }
                } else if (!seen_before && greater < (uint32_t) k) {
                    const int g = atomicAdd(&ax.tie_groups, 1);// at most k groups start below rank k
                    ax.tie_key[g] = my_key;
                    ax.tie_greater[g] = greater;
                    ax.tie_same[g] = same;
                }
            }
            __syncthreads();
            for (int g = warp; g < ax.tie_groups; g += kWarps) {// warp-uniform replay of one group
                const uint32_t gkey = ax.tie_key[g], cap = ax.tie_same[g];
                uint16_t *q = ax.gbuf + ax.tie_greater[g];// this group's slots: [greater, greater + same)
                uint32_t G = 0, sz = 0, head = 0;
                // 32 candidates at a time; only those at or above the group's key are events
                for (int j0 = 0; j0 < m; j0 += 32) {
                    const uint32_t kj = j0 + lane < m ? (uint32_t) ax.fl.key[j0 + lane] : 0u;
                    const uint32_t gt = __ballot_sync(0xffffffffu, kj > gkey);
                    const uint32_t eq = __ballot_sync(0xffffffffu, kj == gkey);
                    // Larger keys between two equal ones act as a run: the first `room` of them (while the
                    // buffer still holds smaller keys to evict) each move the front of the queue to the back,
                    // the others each push the front out.  r rotations of a queue of sz are r mod sz rotations.
                    uint32_t rest = gt, e = eq;
                    while (true) {
                        const int nb = e ? __ffs(e) - 1 : 32;// next equal key in this chunk
                        const uint32_t upto = nb < 32 ? (1u << nb) - 1u : 0xFFFFFFFFu;
                        const uint32_t r = __popc(rest & upto);
                        rest &= ~upto;
                        if (r > 0) {
                            if (sz > 0) {
                                const uint32_t room = (uint32_t) k - (G + sz);// invariant: G + sz <= k
                                const uint32_t rot = r < room ? r : room;
                                uint32_t pops = r - rot;
                                if (sz > 1 && rot > 0) {
                                    const uint32_t rr = rot % sz;
                                    if (sz == cap) {// full ring: turning it is moving the head
                                        head += rr;
                                        if (head >= cap) head -= cap;
                                    } else {
                                        for (uint32_t i = 0; i < rr; ++i) {
                                            uint32_t tail = head + sz;
                                            if (tail >= cap) tail -= cap;
                                            if (lane == 0) q[tail] = q[head];
                                            head = head + 1 == cap ? 0 : head + 1;
                                        }
                                    }
                                }
                                if (pops > sz) pops = sz;
                                head += pops;
                                if (head >= cap) head -= cap;
                                sz -= pops;
                            }
                            G += r;
                        }
                        if (!e) break;
                        e &= e - 1;
                        if (G + sz < (uint32_t) k) {// the equal key joins at the back
                            uint32_t tail = head + sz;
                            if (tail >= cap) tail -= cap;
                            if (lane == 0) q[tail] = (uint16_t) (j0 + nb);
                            ++sz;
                        }
                    }
                }
                __syncwarp();
                for (uint32_t t = lane; t < sz; t += 32) {// G < k whenever sz > 0
                    uint32_t at = head + t;
                    if (at >= cap) at -= cap;
                    ax.top_key[G + t] = gkey;
                    ax.top_idx[G + t] = ax.fl.idx[q[at]];
                }
            }
            __syncthreads();
        } else if (warp == 0) {
            // more ties than the lists hold: stream the whole row through the warp-resident buffer
            TopBuf tb{0, 0, 0, 0};
            for (uint32_t b = 0; b < nblk; ++b) {
                const uint16_t *blk = block_ptr(b);
                const uint32_t gbase = b * kBlk;
                uint32_t w[4], kk[8];
                lds_raw(blk + lane * 8, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) kk[e] = half_at(w, e) == kPad ? 0u : key_of(half_at(w, e));
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
            ax.top_key[lane] = tb.k0;
            ax.top_key[lane + 32] = tb.k1;
            ax.top_idx[lane] = tb.i0;
            ax.top_idx[lane + 32] = tb.i1;
        }
        __syncthreads();
        if (warp < 2) {// exact terms of the top-k, one per thread
            const int i = tid;
            if (i < k) ax.top_term[i] = term_exact(val_of(ax.top_key[i]), val_of(ax.top_key[0]), T);
        }
        __syncthreads();
        if (tid == 0) {
            float sk = 0.f;// the reference's order: one addition after the other
#pragma unroll 1
            for (int i0 = 0; i0 < k; i0 += 4) {
                const float4 q = *reinterpret_cast<const float4 *>(&ax.top_term[i0]);
                sk = __fadd_rn(sk, q.x);
                if (i0 + 1 < k) sk = __fadd_rn(sk, q.y);
                if (i0 + 2 < k) sk = __fadd_rn(sk, q.z);
                if (i0 + 3 < k) sk = __fadd_rn(sk, q.w);
            }
            ax.mail.s_base = sk;
            ax.mail.pos_base = (uint32_t) k;
            ax.mail.mkey = ax.top_key[0];
            ax.mail.done = (uint32_t) k >= n;
        }
        __syncthreads();
        stamp();// 2: top-k in order, top-k terms summed

        if ((uint32_t) k < n) {
            if (!list_ok) {
                if (warp == 0) {
                    // slow path (candidate lists overflowed): one warp walks the leader's part in order
                    minbuf_init(mb, lane, k, raw);
                    if (lane == 0) ax.seg_tau[0] = mb.tau();
                    for (uint32_t b = 0; b < nblk0; ++b) records_direct_block(raw + b * kBlk, b == 0 ? (uint32_t) k : 0u, lane, mb);
                    ax.state[kBounds][lane] = mb.v0 >> 6;
                    ax.state[kBounds][lane + 32] = mb.v1 >> 6;
                    if (lane == 0) ax.seg_tau[kBounds] = mb.tau();
                }
                __syncthreads();
            }
            if (n > n0 && tid < kSlots) ax_of(1u)->state[kBounds][tid] = ax.state[kBounds][tid];// where part 1 starts
        }
        if (tid == 0 && R > 1) ax_of(1u)->seg_tau[kBounds] = ax.seg_tau[kBounds];
        if (tid >= 1 && tid < (int) R) {// hand every helper what it needs
            ax_of((unsigned) tid)->mail.mkey = ax.mail.mkey;
            ax_of((unsigned) tid)->mail.s_base = ax.mail.s_base;
            ax_of((unsigned) tid)->mail.pos_base = ax.mail.pos_base;
            ax_of((unsigned) tid)->mail.done = ax.mail.done;
        }
    }
    cluster.sync();// CS3
    stamp();       // 3: start states known at the leader and the first helper

    // ---- P4: records.  Leader: its segments in parallel, one warp each.  Helpers: one after the other, ----
    // each from the k largest keys its predecessor ends with (the leader's for the first helper), which it
    // hands on in turn.  One cluster barrier per helper that holds data (at least one).
    const unsigned p4_rounds = ranks_used > 2u ? ranks_used - 1u : 1u;
    for (unsigned turn = 1; turn <= p4_rounds; ++turn) {
        if (leader && turn == 1 && list_ok && (uint32_t) k < n) {
            if (warp < kBounds) {// segment i on warp i
                const int sg = warp;
                const uint32_t s_begin = sg == 0 ? (uint32_t) k : kBoundPos[sg - 1];
                if (s_begin < n0) {
                    const int first = ax.rl.seg_first[sg], last = ax.rl.seg_first[sg + 1];
                    MinBuf sb;
                    if (sg == 0) minbuf_init(sb, lane, k, raw);
                    else minbuf_init_keys(sb, lane, k, ax.state[sg]);
                    replay_list(ax.rl.key + first, ax.rl.idx + first, last - first, raw, 0u, lane, sb);
                }
            }
        }
        if (rank == turn && my_n > 0 && !ax.mail.done) {
            const bool have_list = !ax.fl.overflow;
            if (have_list) {
                // the records among this part's list entries: above the k-th largest key of everything before it
                const int cnt = ax.fl.cnt;
                uint32_t my_idx = 0, my_key = 0;
                bool rec = false;
                if (tid < cnt) {
                    my_key = ax.fl.key[tid];
                    my_idx = ax.fl.idx[tid];
                    rec = my_key > ax.seg_tau[kBounds];
                }
                const uint32_t hit_r = __ballot_sync(0xffffffffu, rec);
                if (lane == 0) ax.wcnt_r[warp] = __popc(hit_r);
                __syncthreads();
                const int r_l = ax.wcnt_r[lane];
                const int off_r = __reduce_add_sync(0xffffffffu, lane < warp ? r_l : 0);
                const int cnt_r = __reduce_add_sync(0xffffffffu, r_l);
                if (rec) {
                    const int at = off_r + __popc(hit_r & ((1u << lane) - 1u));
                    ax.rl.key[at] = (uint16_t) my_key;
                    ax.rl.idx[at] = my_idx;
                }
                if (tid == 0) ax.rl.cnt = cnt_r;
                __syncthreads();
            }
            if (warp == 0) {
                MinBuf hb;
                minbuf_init_keys(hb, lane, k, ax.state[kBounds]);
                if (have_list) {
                    replay_list(ax.rl.key, ax.rl.idx, ax.rl.cnt, raw, my_base, lane, hb);
                } else {
                    for (uint32_t b = 0; b < my_nblk; ++b) records_direct_block(raw + b * kBlk, 0u, lane, hb);
                }
                if (rank + 1 < ranks_used) {// the next part starts from what this one ends with
                    Aux *next = ax_of(rank + 1);
                    next->state[kBounds][lane] = hb.v0 >> 6;
                    next->state[kBounds][lane + 32] = hb.v1 >> 6;
                    if (lane == 0) next->seg_tau[kBounds] = hb.tau();
                }
            }
        }
        __syncthreads();// idle warps wait here, at the CTA barrier, for the replaying ones
        cluster.sync();// CS4 (one per turn)
    }
    stamp();       // 4: whole row patched
    M = val_of(ax.mail.mkey);

    // ---- denominator rounds -------------------------------------------------------------
    const float A = kLog2e / T;
    int rounds = 0, replays = 0, int_replays = 0, unsure = 0;
    for (int round = 0; round < kMaxRounds && !ax.mail.done; ++round) {
        ++rounds;
        const float s_base = ax.mail.s_base;
        const uint32_t pos = ax.mail.pos_base;
        const int e0 = (int) ((__float_as_uint(s_base) >> 23) & 0xFFu);
        // z = 2 * term / ulp(s_base) = 2^((v - M) * log2(e) / T + shift); the argument stays below 32
        // in magnitude, so its rounding and the SFU's error keep z within 2^-17.5 (relative) of the truth
        const float shift = (float) (151 - e0);
        const float band = 6.0e-6f;
        const uint32_t gb_first = pos / kBlk;// first global block still to sum
        // block b of this CTA's part is global block b + 256 * rank
        const uint32_t goff = rank * (uint32_t) (kHalfElems / kBlk);
        const uint32_t lb_first = gb_first > goff ? min(gb_first - goff, my_nblk) : 0u;
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
                // Every element is evaluated (no compaction: flagging, scanning and queueing the ones that
                // can contribute costs as many issue slots as evaluating the others too).  z below 1 gives
                // floor 0 and adds nothing; padding and far-away values give z = 0.
                uint32_t w[4];
                lds_raw(raw + b * kBlk + lane * 8, w);
                const uint32_t gpos0 = my_base + b * kBlk + lane * 8;
                const bool partial = my_base + b * kBlk < pos;// only the round's first block
                uint32_t F = 0, Bp = 0, um = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float v = f16_to_f32(half_at(w, e));
                    float arg = fmaf(__fsub_rn(v, M), A, shift);
                    if (partial && gpos0 + e < pos) arg = -1000.f;// already in the running sum
                    const float z = fast_exp2(arg);
                    // floor(z) without the conversion unit (ex2 already keeps it busy): adding 2^23 rounding
                    // down leaves floor(z) in the mantissa; z beyond 2^22 is never "sure" anyway
                    const float t23 = __fadd_rd(fminf(z, 4194304.0f), 8388608.0f);
                    const float fz = t23 - 8388608.0f;
                    // sure when z keeps z * band away from the integers on both sides (never for z >= 0.5 / band)
                    if (fabsf(z - fz - 0.5f) <= fmaf(-z, band, 0.5f)) {
                        const uint32_t f = __float_as_uint(t23) & 0x7FFFFFu;
                        F += f;
                        Bp += ((f & 15u) * 0x00204081u) & 0x01010101u;// bit i of f -> byte i
                    } else {
                        um |= 1u << e;
                    }
                }
                while (um) {// rare: near an integer, or large
                    const int e = __ffs(um) - 1;
                    um &= um - 1;
                    const int slot = atomicAdd(&ax.unc_cnt, 1);
                    if (slot < kUncCap) ax.unc[slot] = b * kBlk + lane * 8 + e;
                    else exact_contrib(ax, b + goff, f16_to_f32(raw[b * kBlk + lane * 8 + e]), M, T, e0);// list full: settle it here
                }
                __syncwarp();
                F = __reduce_add_sync(0xffffffffu, F);
                const uint32_t lo = __reduce_add_sync(0xffffffffu, Bp & 0x00FF00FFu);       // bits 0 and 2
                const uint32_t hi = __reduce_add_sync(0xffffffffu, (Bp >> 8) & 0x00FF00FFu);// bits 1 and 3
                if (lane == 0 && F != 0) {
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
            unsure += ax.unc_cnt;
            for (int i = tid; i < cnt; i += kThreads) {
                const uint32_t lp = ax.unc[i];
                exact_contrib(ax, lp / kBlk + goff, f16_to_f32(raw[lp]), M, T, e0);
            }
        }
        __syncthreads();
        if (!leader) {// ship this helper's block sums to the leader
            for (uint32_t i = tid; i < my_nblk; i += kThreads) {
                const uint32_t g = i + goff;
#pragma unroll
                for (int d = 0; d < kLevels; ++d) lead_ax->C[d][g] = ax.C[d][g];
                lead_ax->tie[g] = ax.tie[g];
            }
        }
        cluster.sync();// CS6
        if (leader) {
            // The walk over the block sums; where the running sum may change binade (or a block holds a
            // half-way case) the block is replayed with real fp32 additions: the CTA evaluates its 256
            // exact terms, one per thread, thread 0 adds them in order, the walk goes on behind the block.
            constexpr uint32_t kNoEvent = 0xFFFFFFFFu;
            uint32_t m = (__float_as_uint(s_base) & 0x7FFFFFu) | 0x800000u;
            int level = 0;
            bool again = false, stop = false;
            float s_cur = s_base;
            uint32_t b0 = gb_first;
            while (true) {
                // One pass over all remaining blocks, 32 per warp: scan inside the warp, chain the warps'
                // totals, find the first block where the sum may carry (or that holds a half-way case).
                {
                    const uint32_t b = b0 + 32u * warp + lane;
                    const bool live = warp < kWalkWarps && b < nblk;
                    const uint32_t rawc = live ? ax.C[level][b] : 0u;
                    const bool tied = live && ((ax.tie[b] >> level) & 1u);
                    uint32_t inc = min(rawc, 1u << 25);// >= 2^24 is a carry by itself; keeps the sums in 32 bits
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
                        if (lane >= o) inc += t;
                    }
                    inc = min(inc, 1u << 25);
                    if (warp < kWalkWarps && lane == 31) ax.walk_tot[warp] = inc;
                    __syncthreads();
                    const uint32_t t_l = lane < kWalkWarps ? ax.walk_tot[lane] : 0u;// at most 16 x 2^25
                    const uint32_t before = __reduce_add_sync(0xffffffffu, lane < warp ? t_l : 0u);
                    const uint32_t all = __reduce_add_sync(0xffffffffu, t_l);
                    const uint32_t m_start = m + min(before, 1u << 25);
                    const uint32_t evm = __ballot_sync(0xffffffffu, tied || (live && m_start + inc >= (1u << 24)));
                    if (warp < kWalkWarps && lane == 0) {
                        const int l = evm ? __ffs(evm) - 1 : -1;
                        ax.walk_ev[warp] = l;
                    }
                    const int l = evm ? __ffs(evm) - 1 : 0;
                    const uint32_t m_at = m_start + (l == 0 ? 0u : __shfl_sync(0xffffffffu, inc, l - 1));
                    if (warp < kWalkWarps && lane == 0) ax.walk_m[warp] = m_at;
                    __syncthreads();
                    // every thread: the first warp with an event
                    const int ev_l = lane < kWalkWarps ? ax.walk_ev[lane] : -1;
                    const uint32_t has = __ballot_sync(0xffffffffu, ev_l >= 0);
                    if (stop || b0 >= nblk || has == 0) {
                        if (!stop && b0 < nblk) {// walked to the end without an event
                            m += all;
                            b0 = nblk;
                        }
                        if (tid == 0) ax.walk_event = kNoEvent;
                    } else {
                        const int w = __ffs(has) - 1;
                        m = ax.walk_m[w];
                        if (tid == 0) ax.walk_event = b0 + 32u * w + (uint32_t) ax.walk_ev[w];
                    }
                }
                __syncthreads();
                const uint32_t eb = ax.walk_event;
                if (eb == kNoEvent) break;
                ++replays;
                // A block that only holds half-way cases (the sum stays inside its binade whatever they round
                // to) is replayed on integers: every element's contribution to the mantissa at this level
                // (from the fast path where that is sure, from the exact term otherwise) is independent of the
                // running value except for the half-way ones, which round to even; those are settled in index
                // order from the prefix sums.  A block in which the sum may carry takes the fp32 replay below.
                if (m + min(ax.C[level][eb], 1u << 25) + (uint32_t) kBlk < (1u << 24)) {
                    ++int_replays;
                    uint32_t c = 0;
                    bool tie = false;
                    if (tid < kBlk) {
                        const uint16_t *blk = block_ptr(eb);
                        const uint32_t j = eb * kBlk + tid;
                        const uint16_t h = blk[tid];
                        if (h != kPad && j >= pos) {
                            const float v = f16_to_f32(h);
                            const float z = fast_exp2(fmaf(__fsub_rn(v, M), A, shift));
                            const float t23 = __fadd_rd(fminf(z, 4194304.0f), 8388608.0f);
                            const float fz = t23 - 8388608.0f;
                            if (fabsf(z - fz - 0.5f) <= fmaf(-z, band, 0.5f)) {// the same test as in the block sums
                                c = ((__float_as_uint(t23) & 0x7FFFFFu) + (1u << level)) >> (level + 1);
                            } else {
                                exact_at_level(term_exact(v, M, T), e0, level, c, tie);
                            }
                        }
                    }
                    uint32_t incl = c;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                        if (lane >= o) incl += t;
                    }
                    const uint32_t tmask = __ballot_sync(0xffffffffu, tie);
                    if (tid < kBlk) {
                        ax.tie_excl[tid] = incl - c;
                        ax.tie_c[tid] = c;
                        if (lane == 31) ax.walk_tot[warp] = incl;
                        if (lane == 0) ax.walk_ev[warp] = (int) tmask;
                    }
                    __syncthreads();
                    if (tid == 0) {
                        uint32_t run = m, adj = 0;// run: mantissa before the current warp's 32 elements, ties not counted
                        for (int w = 0; w < kBlk / 32; ++w) {
                            uint32_t tm = (uint32_t) ax.walk_ev[w];
                            while (tm) {
                                const int l = __ffs(tm) - 1;
                                tm &= tm - 1;
                                const int i = w * 32 + l;
                                // exact value: before + c + 1/2; it rounds up when before + c is odd
                                adj += (run + ax.tie_excl[i] + adj + ax.tie_c[i]) & 1u;
                            }
                            run += ax.walk_tot[w];
                        }
                        ax.walk_m[0] = run + adj;
                    }
                    __syncthreads();
                    m = ax.walk_m[0];
                    b0 = eb + 1;
                    continue;
                }
                if (tid < kBlk) {
                    const uint16_t *blk = block_ptr(eb);
                    const uint32_t j = eb * kBlk + tid;
                    const uint16_t h = blk[tid];
                    ax.blk_terms[tid] = (h == kPad || j < pos) ? 0.f : term_exact(f16_to_f32(h), M, T);
                }
                __syncthreads();
                if (tid == 0) {
                    float s_new = __uint_as_float((uint32_t) (e0 + level - 23) << 23) * (float) m;
                    const float4 *t4 = reinterpret_cast<const float4 *>(ax.blk_terms);
                    float4 q[4] = {t4[0], t4[1], t4[2], t4[3]};// the loads run ahead of the chain of additions
#pragma unroll 1
                    for (int i0 = 0; i0 < kBlk / 4; i0 += 4) {
                        float4 nx[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) nx[u] = t4[min(i0 + 4 + u, kBlk / 4 - 1)];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            s_new = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s_new, q[u].x), q[u].y), q[u].z), q[u].w);
                            q[u] = nx[u];
                        }
                    }
                    ax.walk_s = s_new;
                }
                __syncthreads();
                {// every thread keeps the walk's state
                    const float s_new = ax.walk_s;
                    s_cur = s_new;
                    const int es = (int) ((__float_as_uint(s_new) >> 23) & 0xFFu);
                    level = es - e0;
                    m = (__float_as_uint(s_new) & 0x7FFFFFu) | 0x800000u;
                    b0 = eb + 1;
                    if (level >= kLevels) {
                        again = b0 < nblk;
                        stop = true;
                    }
                }
            }
            if (warp == 0) {
                if (b0 >= nblk && level < kLevels) {
                    s_cur = __uint_as_float((uint32_t) (e0 + level - 23) << 23) * (float) m;
                }
                if (lane == 0) {
                    ax.mail.s_base = s_cur;
                    ax.mail.pos_base = b0 * kBlk;
                    ax.mail.done = again ? 0 : 1;
                    for (unsigned r = 1; r < R; ++r) {
                        ax_of(r)->mail.s_base = s_cur;
                        ax_of(r)->mail.pos_base = b0 * kBlk;
                        ax_of(r)->mail.done = again ? 0 : 1;
                    }
                }
            }
        }
        __syncthreads();
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
                dbg[129 + 14] = (float) replays;
                dbg[129 + 13] = (float) unsure;
                dbg[129 + 12] = (float) int_replays;
            }
            uint64_t *slot = a.result + (int64_t) row * a.result_stride;
            pick_from_topk(ax.top_term, ax.top_idx, k, a.topp, random_val, slot);
            if (pr.world) {
                // the index to every rank's results; the row that reports last closes the call for this rank: "done"
                // to every peer, wait for theirs (then all rows are local and nobody reads this rank's shard any more)
                const unsigned long long picked = *slot;
                for (uint32_t p = 0; p < pr.world; ++p) {
                    if (p != pr.rank) peer_st_u64(pr.results[p] + pr.row0 + row, picked);
                }
                __threadfence_system();
                uint32_t *mine = pr.flags[pr.rank];
                if (atomicAdd(&mine[kPeerFinished], 1u) == pr.rows - 1) {
                    mine[kPeerFinished] = 0;
                    __threadfence_system();
                    for (uint32_t p = 0; p < pr.world; ++p) peer_st_release(&pr.flags[p][kPeerDone + pr.rank], peer_call);
                    for (uint32_t p = 0; p < pr.world; ++p) peer_wait(&mine[kPeerDone + p], peer_call);
                    mine[kPeerCalls] = peer_call;
                }
            }
        }
    }
}

}// namespace

namespace b200 {

// Sampling branch for rows of at most 262144 logits and topk <= 64: one CTA per row up to 65536 logits, a
// cluster of two up to 131072, of four beyond.
bool random_sample_pair_supported(int voc) { return voc >= 1 && voc <= kMaxRanks * kHalfElems; }

unsigned long long random_sample_pair_timeouts_read() {
    unsigned long long v = 0;
    if (cudaMemcpyFromSymbol(&v, g_pair_peer_timeouts, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return ~0ull;
    }
    return v;
}

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
    // one CTA per row while the row fits it: a second one would only occupy an SM another row could use
    const unsigned ranks = a.voc > 2 * kHalfElems ? 4u : a.voc > kHalfElems ? 2u : 1u;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ranks * (unsigned) rows);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, random_sample_pair_kernel, a);
    return check_launch("random_sample_pair");
}

}// namespace b200
