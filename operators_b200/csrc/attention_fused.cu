// Attention with several new tokens per call in ONE kernel: the scores of a block of 128 query rows never leave the
// SM.
//
// The reference composite (src/ops/attention/operator.cc:252-305) materialises the fp16 score tensor
// [n_q_head, seq, total] between its two matmuls; at 4096 x 4096 tokens that tensor (1 GB written, read, written
// and read again) sets the pace, not the tensor cores.  Here a CTA owns 128 query rows of one q head and walks the
// visible cached tokens in tiles of 64, twice:
//   pass 1  S = q k^T on tcgen05.mma into tensor memory; the softmax warps (two threads per query row = TMEM lane)
//           read S, round alpha * s to fp16 as the reference's score tensor holds it, and keep the row's running
//           maximum and sum of exponentials;
//   pass 2  S again (the tensor pipe has time to spare: the exponentials bound the kernel), the probability
//           exp(s - max) / sum truncated to fp16 exactly as the causal softmax stores it, written as the K-major A
//           operand into 128-byte-swizzled shared memory, and O += P v on tcgen05.mma with v read as an MN-major B
//           operand straight from the cache rows; O stays in tensor memory over the whole pass.
// The epilogue truncates O to fp16 and writes out[row, head, :], which is the reference's closing rearrange.
// Because the maximum and the sum are final before any probability is formed, O needs no rescaling and every value
// that the reference rounds (score, probability, output) is rounded at the same place; only the grouping of the
// fp32 sums differs.
//
// Roles (320 threads, two CTAs per SM so that one CTA's exponentials overlap the other's products):
//   warps 0-7  softmax / epilogue: two threads per query row, 32 of a tile's 64 columns each; warp w owns TMEM
//              lanes 32 (w & 3) .. + 31; the halves of a row exchange maximum and sum once, between the passes
//   warp 8     one lane issues the TMA loads: q once, then k tiles (both passes) and v tiles (pass 2) through one
//              ring of shared-memory slots, as far ahead as the ring is long
//   warp 9     allocates TMEM (S twice 64 columns, O dh columns); one lane issues the MMAs.  S of tile j + 2 is
//              issued before P v of tile j (its buffer is free once S of tile j has been read), so the softmax
//              warps find their next scores ready.
// Calls of fewer than 128 tokens with several q heads per kv head: a block holds 128 / group tokens of all q heads
// of one kv head (row = token * group + head), loaded by one TMA box [tokens][heads][64], so the block is full and k
// and v are loaded once per kv head.
// Head sizes: multiples of 8 up to 256; the 64-element boxes read what lies beyond the head size as zeros (DHB boxes;
// beyond 128 a CTA takes all 512 TMEM columns and an SM to itself).
// Few blocks of query rows over many cached tokens (a chunk of a prompt, speculative drafts): up to 8 CTAs, one
// thread-block cluster, share a block and each takes a range of its tiles.  After pass 1 they exchange their rows'
// maximum and sum over distributed shared memory (one mbarrier per CTA that every CTA of the cluster arrives on; the
// waits acquire at cluster scope), after pass 2 each parks its fp32 partial of O in its shared memory and CTA r
// adds its share of the rows of all partials in rank order, truncates and stores them.  A CTA whose range is empty
// (the first rows of a prompt see fewer tiles than the cluster has CTAs) contributes -inf, 0 and zeros.
// Every mbarrier wait is bounded (tc_ptx.cuh); a role that gives up raises the CTA's abort flag, all roles leave,
// copies in flight are awaited (bounded), TMEM is freed, and infiniopExtDeviceTimeouts reports it.
#include "attention_prefill.cuh"
#include "tc_ptx.cuh"

#include <mutex>
#include <new>
#include <type_traits>

namespace b200 {

namespace {

using namespace tc;

constexpr int kSoftmaxThreads = 256;                 // two threads per query row, 32 of a tile's 64 columns each
constexpr int kFusedThreads = kSoftmaxThreads + 64;  // + the warp that loads and the warp that issues the MMAs
constexpr uint32_t kRows = 128;// query rows per CTA = TMEM lanes
constexpr uint32_t kKeys = 64; // cached tokens per tile: one 128-byte swizzle row of P
// TMEM columns: S0 [0, 64), S1 [64, 128), O [128, 128 + 64 * DHB); a power of two, so 256 up to dh 128 (two CTAs per
// SM) and all 512 beyond (one CTA per SM)
__host__ __device__ constexpr uint32_t tmem_cols(int dhb) { return dhb <= 2 ? 256u : 512u; }
constexpr uint32_t kMinSmem = 80 * 1024;// keeps a third CTA (and its TMEM request) off the SM

struct FusedParams {
    uint32_t nh, group, seq, total, tiles_m;
    uint32_t dh;// head size, a multiple of 8 up to 64 * DHB: the boxes read the elements beyond it as zeros
    uint32_t slots;// k / v tiles of the shared-memory ring (4 when two CTAs share an SM, more for a CTA alone)
    uint32_t splits;// CTAs (one cluster) that share a block of query rows, each with a range of the cached tokens
    // Rows of a block: 128 tokens of one q head (pack = 1), or, for calls of few tokens, tok tokens of all `pack` q
    // heads of one kv head (row = token * pack + head within the group), so that the block is full and k / v are
    // loaded once per kv head.  tiles_m counts the blocks of tokens either way.
    uint32_t pack, tok;
    float alpha;
    uint16_t *out;// [seq, nh, dh]
};

constexpr uint32_t kMaxSlots = 16;// k / v tiles in flight per CTA
constexpr float kExactFrom = 1024.f;// row maxima from here on: x - max formed before the multiplication by log2(e)
constexpr uint32_t kMaxSplits = 8;// CTAs of a cluster that share a block of query rows (the portable cluster size)
// Waiting roles sleep in the barrier instead of polling: twenty warps share an SM and the exponentials need the issue
// slots (polling producer and MMA lanes took four of ten issued instructions).
constexpr uint32_t kSuspendNs = 20000;

// Development aid (-DB200_ATTN_FUSED_TRACE): thread 0 of CTA 0 adds up the clock ticks it spends in each step of the
// softmax loops.  Not compiled into the library.
#ifdef B200_ATTN_FUSED_TRACE
__device__ unsigned long long g_attn_trace[16];
#define TRACE_NOW(var) const long long var = clock64()
#define TRACE_ADD(slot, t0, t1) \
    if (threadIdx.x == 0 && blockIdx.x == 0) g_attn_trace[slot] += (unsigned long long) ((t1) - (t0))
#else
#define TRACE_NOW(var)
#define TRACE_ADD(slot, t0, t1)
#endif
// barriers: the ring's full / empty pairs first
enum Bar { kFull = 0, kEmpty = kMaxSlots, kQFull = 2 * kMaxSlots, kSFull, kSFull1, kSEmpty, kSEmpty1, kPFull, kPEmpty, kOFull,
           kStatsFull, kStatsRead, kOStaged,// between the CTAs of a cluster (splits > 1): one arrival per CTA
           kBars };

__device__ __forceinline__ uint32_t hmax2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hmin2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("min.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// 32 scores of one query row (columns col0 .. col0 + 31 of the score matrix) as the reference's fp16 score tensor
// holds them, two per word: alpha * s truncated to fp16, columns beyond vis_last at -inf.  The packed conversion
// saturates where the reference's rule (common.cuh f32_to_f16_ref) produces its overflow patterns, so in pass 1
// (CHECK) a chunk whose extreme values reach the largest finite fp16 is redone element by element with that rule
// and `exact` stays set for the rest of the row's columns of this thread; pass 2 converts the same elements again
// and only reads the flag.
template<bool CHECK>
__device__ __forceinline__ void pack_scores(const float *s, uint32_t *w, float alpha, uint32_t col0, uint32_t vis_last, bool &exact) {
    uint32_t hi = 0xFC00FC00u, lo = 0x7C007C00u;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(w[i]) : "f"(__fmul_rn(alpha, s[2 * i + 1])), "f"(__fmul_rn(alpha, s[2 * i])));
        if (CHECK) hi = hmax2_u32(hi, w[i]), lo = hmin2_u32(lo, w[i]);
    }
    const uint32_t big = 0x7BFFu;
    if (CHECK && ((hi & 0xFFFFu) == big || (hi >> 16) == big || (lo & 0xFFFFu) == (big | 0x8000u) || (lo >> 16) == (big | 0x8000u))) {
        exact = true;
    }
    if (exact) {
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = pack2_ref(__fmul_rn(alpha, s[2 * i]), __fmul_rn(alpha, s[2 * i + 1]));
    }
    if (col0 + 31 > vis_last) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t c = col0 + 2 * i;
            if (c > vis_last) w[i] = 0xFC00FC00u;
            else if (c + 1 > vis_last) w[i] = (w[i] & 0xFFFFu) | 0xFC000000u;
        }
    }
}

template<int DHB>// dh / 64
__global__ void __launch_bounds__(kFusedThreads, 2)
    attn_fused_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const FusedParams p) {
    constexpr uint32_t kQBytes = DHB * kRows * 128u;// DHB boxes of 128 rows x 64 elements
    constexpr uint32_t kKVBytes = DHB * kKeys * 128u;// DHB boxes of 64 rows x 64 elements
    constexpr uint32_t kPBytes = kRows * kKeys * 2u;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // q | ring of k / v tiles | P | barriers.  The swizzled tiles need 1024-byte alignment; the request leaves no room
    // to round the base up (two CTAs fill the SM), so a base that is not aligned ends the CTA before it starts.
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicAdd(&g_tc_gemm_timeouts, 1ull);
        return;
    }
    unsigned char *sq = smem_raw, *ring = sq + kQBytes, *sp = ring + p.slots * kKVBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sp + kPBytes);
    float2 *ml = reinterpret_cast<float2 *>(sp);// [2][128]: each half's maximum and sum of a row, between the passes
    float2 *ml_cta = ml + 2 * kRows;           // [128]: this CTA's maximum and sum of a row, read by its cluster
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the longest blocks (last query rows) start first
    const uint32_t S = p.splits, split = S > 1 ? cluster_rank() : 0u, unit = blockIdx.x / S;
    const uint32_t heads = p.pack > 1 ? p.nh / p.group : p.nh;// blocks per block of tokens: kv heads when packed
    const uint32_t tm = p.tiles_m - 1 - unit / heads, hb = unit % heads;
    const uint32_t h0 = p.pack > 1 ? hb * p.group : hb, kvh = h0 / p.group;// first (or only) q head of the block
    const uint32_t tok0 = tm * p.tok;                                       // first token of the block
    const uint32_t last_tok = min(tok0 + p.tok - 1, p.seq - 1);
    const uint32_t tiles_all = (p.total - p.seq + last_tok) / kKeys + 1;// tiles that hold a visible column
    // this CTA's share of them (possibly none): its maxima, sums and outputs meet the other CTAs' over distributed
    // shared memory
    const uint32_t t_begin = split * tiles_all / S, tiles = (split + 1) * tiles_all / S - t_begin;

    if (threadIdx.x == 0) {
        for (int b = 0; b < kBars; ++b) {
            const bool softmax_arrives = b == kSEmpty || b == kSEmpty1 || b == kPFull;
            const bool ctas_arrive = b == kStatsFull || b == kStatsRead || b == kOStaged;
            mbar_init(&bars[b], softmax_arrives ? (uint32_t) kSoftmaxThreads : ctas_arrive ? S : 1u);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, tmem_cols(DHB));
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    if (S > 1) cluster_sync_all();// nobody arrives on a barrier of another CTA before it exists
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // one box per 64 head elements: [128 tokens] of head h0, or [tok tokens][pack heads] (the map's box)
            mbar_expect_tx(&bars[kQFull], DHB * p.tok * p.pack * 128u);
            for (int kb = 0; kb < DHB; ++kb) {
                if (p.pack > 1) tma_load_3d(sq + kb * (kRows * 128u), &map_q, &bars[kQFull], kb * 64, (int32_t) h0, (int32_t) tok0);
                else tma_load_3d(sq + kb * (kRows * 128u), &map_q, &bars[kQFull], kb * 64, (int32_t) tok0, (int32_t) h0);
            }
            // the caches are complete once the append kernel ahead of this one has finished (q does not depend on it)
            asm volatile("griddepcontrol.wait;" ::: "memory");
            // The ring is a queue: tiles are loaded in the order in which the MMA lane uses them.  Pass 1: k(0) ..
            // k(T - 1); pass 2: k(0), k(1), then k(j + 2), v(j) for j = 0 .. T - 1.
            uint32_t slot = 0, ph = 0;
            auto load = [&](bool is_v, uint32_t j) -> bool {
                if (!mbar_wait<kSuspendNs>(&bars[kEmpty + slot], ph ^ 1u, abort_flag)) return false;
                mbar_expect_tx(&bars[kFull + slot], kKVBytes);
                for (int x = 0; x < DHB; ++x) {// k: 64 of the dh elements per box (K-major); v: the same boxes (MN-major)
                    tma_load_3d(ring + slot * kKVBytes + x * (kKeys * 128u), is_v ? &map_v : &map_k, &bars[kFull + slot], x * 64,
                                (int32_t) (j * kKeys), (int32_t) kvh);
                }
                if (++slot == p.slots) slot = 0, ph ^= 1u;
                return true;
            };
            bool ok = true;
            for (uint32_t n = 0; ok && n < tiles; ++n) ok = load(false, t_begin + n);
            for (uint32_t n = 0; ok && n < 2 && n < tiles; ++n) ok = load(false, t_begin + n);
            for (uint32_t j = 0; ok && j < tiles; ++j) {
                if (j + 2 < tiles) ok = load(false, t_begin + j + 2);
                if (ok) ok = load(true, t_begin + j);
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc(kRows, kKeys, 0, 0), idesc_o = make_idesc(kRows, DHB * 64, 0, 1);
            const uint32_t aq = smem_u32(sq), aring = smem_u32(ring), ap = smem_u32(sp);
            uint32_t slot = 0, slot_ph = 0;// the ring slot of the next tile in the producer's order
            // S(n) = q k(n)^T into S buffer n & 1: waits for the k tile and for the softmax warps to have read S(n - 2)
            auto issue_s = [&](uint32_t n) -> bool {
                const uint32_t b = n & 1u, ph = (n >> 1) & 1u;
                if (!mbar_wait<kSuspendNs>(&bars[kFull + slot], slot_ph, abort_flag)) return false;
                if (!mbar_wait<kSuspendNs>(&bars[kSEmpty + b], ph ^ 1u, abort_flag)) return false;
                tc_fence_after();
#pragma unroll
                for (int kb = 0; kb < DHB; ++kb) {
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint64_t da = make_smem_desc(aq + kb * (kRows * 128u) + i * 32u, 16, 1024);
                        const uint64_t db = make_smem_desc(aring + slot * kKVBytes + kb * (kKeys * 128u) + i * 32u, 16, 1024);
                        umma_f16(tmem_base + b * kKeys, da, db, idesc_s, (kb > 0 || i > 0) ? 1u : 0u);
                    }
                }
                umma_commit(&bars[kEmpty + slot]);
                umma_commit(&bars[kSFull + b]);
                if (++slot == p.slots) slot = 0, slot_ph ^= 1u;
                return true;
            };
            bool ok = mbar_wait<kSuspendNs>(&bars[kQFull], 0, abort_flag);
            uint32_t n = 0;
            for (; ok && n < tiles; ++n) ok = issue_s(n);// pass 1
            for (uint32_t j = 0; ok && j < 2 && j < tiles; ++j) ok = issue_s(n++);// pass 2, tiles 0 and 1
            for (uint32_t j = 0; ok && j < tiles; ++j) {
                // S of tile j + 2 goes first: its buffer is free as soon as the softmax warps have read S of tile j,
                // long before they deliver P of tile j, so no product waits behind the exponentials
                if (j + 2 < tiles) {
                    ok = issue_s(n++);
                    if (!ok) break;
                }
                if (!mbar_wait<kSuspendNs>(&bars[kPFull], j & 1u, abort_flag) || !mbar_wait<kSuspendNs>(&bars[kFull + slot], slot_ph, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    // P: K-major, 16 keys = 32 bytes along the swizzled rows; v: MN-major, 16 keys = 16 rows of 128
                    // bytes, the second 64 head elements one box further
                    const uint64_t da = make_smem_desc(ap + i * 32u, 16, 1024);
                    const uint64_t db = make_smem_desc(aring + slot * kKVBytes + i * 2048u, kKeys * 128u, 1024);
                    umma_f16(tmem_base + 2 * kKeys, da, db, idesc_o, (j > 0 || i > 0) ? 1u : 0u);
                }
                umma_commit(&bars[kPEmpty]);
                umma_commit(&bars[kEmpty + slot]);
                if (++slot == p.slots) slot = 0, slot_ph ^= 1u;
                if (j + 1 == tiles) umma_commit(&bars[kOFull]);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax and epilogue (warps 0..7)
        // warp w reads TMEM lanes 32 (w & 3) .. + 31 (the lanes a warp may touch follow from its index) and the
        // columns 32 (w >> 2) .. + 31 of every tile
        const uint32_t quarter = warp & 3u, half = warp >> 2;
        const uint32_t lane_row = quarter * 32 + lane;
        const uint32_t row = tok0 + lane_row / p.pack, head = h0 + lane_row % p.pack;// this row's token and q head
        const bool row_valid = row < p.seq && lane_row < p.tok * p.pack;
        const uint32_t vis_last = p.total - p.seq + row;// last visible column of this row
        const uint32_t t_lane = tmem_base + ((quarter * 32u) << 16);
        float m = -INFINITY, l = 0.f;
        bool exact = false, ok = true;
        uint32_t w[16];
        // this thread's 32 scores of tile j (S index n), packed
        auto load_scores = [&](uint32_t n, uint32_t j, auto first_pass) -> bool {
            const uint32_t b = n & 1u;
            [[maybe_unused]] constexpr int kT = decltype(first_pass)::value ? 0 : 4;
            TRACE_NOW(t0);
            if (!mbar_wait<kSuspendNs>(&bars[kSFull + b], (n >> 1) & 1u, abort_flag)) return false;
            TRACE_NOW(t1);
            tc_fence_after();
            float s[32];
            tmem_ld32(t_lane + b * kKeys + half * 32u, s);
            tc_fence_before();
            mbar_arrive(&bars[kSEmpty + b]);
            TRACE_NOW(t2);
            pack_scores<decltype(first_pass)::value>(s, w, p.alpha, j * kKeys + half * 32u, vis_last, exact);
            TRACE_NOW(t3);
            TRACE_ADD(kT + 0, t0, t1);
            TRACE_ADD(kT + 1, t1, t2);
            TRACE_ADD(kT + 2, t2, t3);
            return true;
        };
#pragma unroll 1
        for (uint32_t n = 0; n < tiles; ++n) {// pass 1: maximum and sum over this thread's columns of the row
            if (!(ok = load_scores(n, t_begin + n, std::true_type{}))) break;
            TRACE_NOW(ta);
            uint32_t t8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t8[i] = hmax2_u32(w[i], w[i + 8]);
#pragma unroll
            for (int i = 0; i < 4; ++i) t8[i] = hmax2_u32(t8[i], t8[i + 4]);
            const float2 mt = unpack2(hmax2_u32(hmax2_u32(t8[0], t8[1]), hmax2_u32(t8[2], t8[3])));
            const float m_new = fmaxf(m, fmaxf(mt.x, mt.y));
            // exp(x - m) as 2^(x log2e - m log2e) in one multiply-add: the product m log2e is rounded, an error of
            // |m| 2^-24 in the exponent, nothing for ordinary scores; a warp that holds a row with a maximum beyond
            // kExactFrom forms x - m first (exact: both are fp16 values), one more instruction per score
            const bool far = __any_sync(0xffffffffu, m_new != -INFINITY && fabsf(m_new) >= kExactFrom);
            if (m_new != -INFINITY) {// else: all of this thread's columns so far are masked
                float part[4] = {0.f, 0.f, 0.f, 0.f};
                if (!far) {
                    const float mk = -m_new * kLog2e;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 f = unpack2(w[i]);
                        part[(2 * i) & 3] += fast_exp2(fmaf(f.x, kLog2e, mk));
                        part[(2 * i + 1) & 3] += fast_exp2(fmaf(f.y, kLog2e, mk));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 f = unpack2(w[i]);
                        part[(2 * i) & 3] += fast_exp2((f.x - m_new) * kLog2e);
                        part[(2 * i + 1) & 3] += fast_exp2((f.y - m_new) * kLog2e);
                    }
                }
                const float scale = m == -INFINITY ? 0.f : fast_exp2((m - m_new) * kLog2e);
                l = fmaf(l, scale, (part[0] + part[1]) + (part[2] + part[3]));
                m = m_new;
            }
            TRACE_NOW(tb);
            TRACE_ADD(3, ta, tb);
        }
        // the two halves of a row meet: (m, l) of the whole row
        ml[half * kRows + lane_row] = make_float2(m, l);
        asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
        {
            const float2 o = ml[(half ^ 1u) * kRows + lane_row];
            // (column 0 is visible to every row, so the maximum is finite in the CTA that holds tile 0; a CTA whose
            // tiles are all masked for a row, or that has no tiles, carries -inf and 0)
            const float m_all = fmaxf(m, o.x);
            const float mine = m == -INFINITY ? 0.f : l * fast_exp2((m - m_all) * kLog2e);
            const float theirs = o.x == -INFINITY ? 0.f : o.y * fast_exp2((o.x - m_all) * kLog2e);
            l = half == 0 ? mine + theirs : theirs + mine;// the same sum in both threads
            m = m_all;
        }
        if (S > 1) {
            // the CTAs of the cluster meet: every CTA publishes its rows' (m, l), raises a barrier in every CTA, and
            // combines all of them in rank order (the same bits everywhere)
            if (half == 0) ml_cta[lane_row] = make_float2(m, l);
            asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
            if (threadIdx.x == 0) {
                for (uint32_t r = 0; r < S; ++r) mbar_arrive_remote(mapa_u32(smem_u32(&bars[kStatsFull]), r));
            }
            if (ok) ok = mbar_wait_cluster(&bars[kStatsFull], 0, abort_flag);
            if (ok) {
                const uint32_t mine_addr = smem_u32(&ml_cta[lane_row]);
                float m_all = -INFINITY;
                float2 part[kMaxSplits];
#pragma unroll
                for (uint32_t r = 0; r < kMaxSplits; ++r) {
                    part[r] = r < S ? ld_cluster_f2(mapa_u32(mine_addr, r)) : make_float2(-INFINITY, 0.f);
                    m_all = fmaxf(m_all, part[r].x);
                }
                float l_all = 0.f;
#pragma unroll
                for (uint32_t r = 0; r < kMaxSplits; ++r) {
                    if (part[r].x != -INFINITY) l_all += part[r].y * fast_exp2((part[r].x - m_all) * kLog2e);
                }
                m = m_all, l = l_all;
            }
            // nobody overwrites its (m, l) with P before every CTA has read them
            asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
            if (threadIdx.x == 0) {
                for (uint32_t r = 0; r < S; ++r) mbar_arrive_remote(mapa_u32(smem_u32(&bars[kStatsRead]), r));
            }
            if (ok) ok = mbar_wait_cluster(&bars[kStatsRead], 0, abort_flag);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");// the exchange area becomes P again
        // exp(x - m) / l as one exponential: 2^(x log2e - m log2e - log2 l), or 2^((x - m) log2e - log2 l) for a warp that
        // holds a row with a distant maximum (see pass 1)
        const float log2l = log2f(l), mk = fmaf(-m, kLog2e, -log2l);
        const bool far = __any_sync(0xffffffffu, fabsf(m) >= kExactFrom);
#pragma unroll 1
        for (uint32_t j = 0; ok && j < tiles; ++j) {// pass 2: probabilities into shared memory for P v
            if (!(ok = load_scores(tiles + j, t_begin + j, std::false_type{}))) break;
            TRACE_NOW(ta);
            if (!far) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 f = unpack2(w[i]);
                    asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(w[i]) : "f"(fast_exp2(fmaf(f.y, kLog2e, mk))), "f"(fast_exp2(fmaf(f.x, kLog2e, mk))));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 f = unpack2(w[i]);
                    asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(w[i])
                        : "f"(fast_exp2(fmaf(f.y - m, kLog2e, -log2l))), "f"(fast_exp2(fmaf(f.x - m, kLog2e, -log2l))));
                }
            }
            TRACE_NOW(tb);
            if (!(ok = mbar_wait<kSuspendNs>(&bars[kPEmpty], (j & 1u) ^ 1u, abort_flag))) break;
            TRACE_NOW(tc_);
            // row r of the K-major operand: 128 bytes, 16-byte chunk c at position c ^ (r & 7) (128-byte swizzle)
            unsigned char *prow = sp + lane_row * 128u;
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c) {
                *reinterpret_cast<uint4 *>(prow + (((half * 4 + c) ^ (lane_row & 7u)) << 4)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");// the MMA reads P through the async proxy
            mbar_arrive(&bars[kPFull]);
            TRACE_NOW(td);
            TRACE_ADD(7, ta, tb);
            TRACE_ADD(8, tb, tc_);
            TRACE_ADD(9, tc_, td);
        }
        constexpr uint32_t kCols = DHB * 32;// this thread's half of the row's dh outputs
        if (S == 1) {
            if (ok && mbar_wait<kSuspendNs>(&bars[kOFull], 0, abort_flag)) {
                tc_fence_after();
                uint16_t *orow = p.out + ((size_t) row * p.nh + head) * p.dh + half * kCols;
#pragma unroll
                for (uint32_t c0 = 0; c0 < kCols; c0 += 16) {
                    float acc[16];
                    tmem_ld16(t_lane + 2 * kKeys + half * kCols + c0, acc);// every lane takes part in the load
                    uint32_t o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = pack2_ref(acc[2 * i], acc[2 * i + 1]);
                    if (row_valid) {// (columns beyond dh are the zero padding of v)
                        uint4 *dst = reinterpret_cast<uint4 *>(orow + c0);
                        if (half * kCols + c0 < p.dh) dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                        if (half * kCols + c0 + 8 < p.dh) dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                }
            }
        } else {
            // Every CTA parks its fp32 partial of O in its shared memory (q and the ring are idle by now; row r's
            // 16-byte groups at position g ^ (r % 16), so that a warp's stores spread over the banks), the
            // cluster meets, and CTA `split` adds rows [split * 128 / S, ...) of all partials in rank order,
            // truncates and stores them.
            constexpr uint32_t kGroups = DHB * 16;// float4 groups per row
            float4 *stage = reinterpret_cast<float4 *>(sq);
            const bool have = tiles > 0;
            if (have && ok) ok = mbar_wait<kSuspendNs>(&bars[kOFull], 0, abort_flag);
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (uint32_t c0 = 0; c0 < kCols; c0 += 16) {
                    float acc[16];
                    if (have) tmem_ld16(t_lane + 2 * kKeys + half * kCols + c0, acc);// uniform over the CTA
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint32_t g = (half * kCols + c0) / 4 + i;
                        stage[lane_row * kGroups + (g ^ (lane_row & 15u))] =
                            have ? make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
            if (threadIdx.x == 0) {
                for (uint32_t r = 0; r < S; ++r) mbar_arrive_remote(mapa_u32(smem_u32(&bars[kOStaged]), r));
            }
            if (ok) ok = mbar_wait_cluster(&bars[kOStaged], 0, abort_flag);
            if (ok) {
                const uint32_t rows_per = (kRows + S - 1) / S, r_first = min(split * rows_per, kRows);
                const uint32_t rows_mine = min(rows_per, kRows - r_first);
                for (uint32_t idx = threadIdx.x; idx < rows_mine * kGroups; idx += kSoftmaxThreads) {
                    const uint32_t r = r_first + idx / kGroups, g = idx % kGroups;
                    const uint32_t addr = smem_u32(&stage[r * kGroups + (g ^ (r & 15u))]);
                    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (uint32_t c = 0; c < S; ++c) {
                        const float4 v = ld_cluster_f4(mapa_u32(addr, c));
                        sum.x += v.x, sum.y += v.y, sum.z += v.z, sum.w += v.w;
                    }
                    const uint32_t tok = tok0 + r / p.pack;
                    if (tok < p.seq && r < p.tok * p.pack && g * 4 < p.dh) {
                        uint2 *dst = reinterpret_cast<uint2 *>(p.out + ((size_t) tok * p.nh + h0 + r % p.pack) * p.dh + g * 4);
                        *dst = make_uint2(pack2_ref(sum.x, sum.y), pack2_ref(sum.z, sum.w));
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // let TMA copies that are still in flight land before the shared memory is given back
        for (uint32_t i = 0; i <= p.slots; ++i) {
            uint64_t *bar = i < p.slots ? &bars[kFull + i] : &bars[kQFull];
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, 0) && !mbar_try_wait(bar, 1) && clock64() - t0 < 2000000ll) {}
        }
    }
    __syncthreads();
    if (S > 1) cluster_sync_all();// no CTA leaves while another may still read its shared memory
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols(DHB));
    }
}

using FusedKernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const FusedParams);
FusedKernel fused_kernel(uint32_t dhb) {
    return dhb == 1 ? attn_fused_kernel<1> : dhb == 2 ? attn_fused_kernel<2> : dhb == 3 ? attn_fused_kernel<3> : attn_fused_kernel<4>;
}

// Shared memory of a CTA with `slots` ring tiles.
size_t fused_smem_bytes(uint32_t dhb, uint32_t slots) {
    const size_t need = (size_t) dhb * kRows * 128 + (size_t) slots * dhb * kKeys * 128 + kRows * kKeys * 2 + kBars * 8 + 16;
    return need < kMinSmem ? kMinSmem : need;
}
// The most ring tiles that fit `budget` bytes (at most kMaxSlots); 0 when not even four fit.
uint32_t fused_slots(uint32_t dhb, size_t budget) {
    uint32_t slots = kMaxSlots;
    while (slots >= 4 && fused_smem_bytes(dhb, slots) > budget) --slots;
    return slots >= 4 ? slots : 0;
}

}// namespace

struct AttnFused {
    int device_id;
    AttnPrefillShape shape;
    uint32_t dhb, tiles_m, slots, splits, pack, tok;
    size_t smem_bytes;
    std::mutex mu;
    bool valid = false;
    const void *q_ptr = nullptr, *k_ptr = nullptr, *v_ptr = nullptr;
    CUtensorMap map_q, map_k, map_v;
};

// Blocks of query rows: few tokens per call and several q heads per kv head -> the heads of a group share a block.
static void fused_blocks(const AttnPrefillShape &s, uint32_t &pack, uint32_t &tok, uint64_t &blocks) {
    pack = (s.group > 1 && s.group <= kRows && s.seq < kRows) ? s.group : 1u;
    tok = kRows / pack;
    blocks = (uint64_t) ((s.seq + tok - 1) / tok) * (pack > 1 ? s.nh / s.group : s.nh);
}

static bool encode_maps(AttnFused *f, const void *q, const void *k_cache, const void *v_cache) {
    const AttnPrefillShape &s = f->shape;
    const uint32_t nkvh = s.nh / s.group;
    // rows beyond seq / total read as zeros: the caches' unused rows are never touched
    const bool q_ok = f->pack > 1
        ? tc_encode_tiles_f16(&f->map_q, q, s.dh, s.nh, s.seq, (uint64_t) s.q_s0 * 2, (uint64_t) s.q_s1 * 2, f->pack, f->tok)
        : tc_encode_tiles_f16(&f->map_q, q, s.dh, s.seq, s.nh, (uint64_t) s.q_s1 * 2, (uint64_t) s.q_s0 * 2, kRows);
    return q_ok &&
           tc_encode_tiles_f16(&f->map_k, k_cache, s.dh, s.total, nkvh, (uint64_t) s.kc_s1 * 2, (uint64_t) s.kc_s0 * 2, kKeys) &&
           tc_encode_tiles_f16(&f->map_v, v_cache, s.dh, s.total, nkvh, (uint64_t) s.vc_s1 * 2, (uint64_t) s.vc_s0 * 2, kKeys);
}

// Few blocks of query rows over many cached tokens: up to 8 CTAs (one cluster) share a block and split its tokens, as
// long as all CTAs still run at once (two per SM) and every CTA keeps at least four tiles.  Doubling finds the size;
// when the hardware cannot hold that many clusters of that size at once (a cluster needs its SMs in one GPC: 15
// clusters of 8 CTAs, where 16 blocks wanted 16), a slightly smaller cluster that runs them all in one go is better
// than a second round.
uint32_t attn_fused_splits(const AttnPrefillShape &s, int sm_count, int device_id) {
    uint32_t pack, tok;
    uint64_t ctas;
    fused_blocks(s, pack, tok, ctas);
    const uint64_t kv_tiles = (s.total + kKeys - 1) / kKeys;
    uint32_t splits = 1;
    const uint32_t dhb = (s.dh + 63) / 64;
    const uint64_t places = (uint64_t) sm_count * (dhb <= 2 ? 2 : 1);// CTAs that run at once
    while (splits < kMaxSplits && ctas * splits * 2 <= places && kv_tiles >= 8ull * splits) splits *= 2;
    if (splits <= 2 || s.dh % 8 != 0 || s.dh > 256) return splits;
    DeviceGuard guard(device_id);
    int sm_bytes = 0;
    if (cudaDeviceGetAttribute(&sm_bytes, cudaDevAttrMaxSharedMemoryPerMultiprocessor, device_id) != cudaSuccess) {
        cudaGetLastError();
        return splits;
    }
    FusedKernel kernel = fused_kernel(dhb);
    const uint32_t slots_alone = fused_slots(dhb, (size_t) sm_bytes - 1024), slots_shared = fused_slots(dhb, (size_t) sm_bytes / 2 - 1024);
    // (the attribute is the most any launch of the kernel may ask for: never lower it for the query)
    if (slots_alone == 0 ||
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) fused_smem_bytes(dhb, slots_alone)) != cudaSuccess) {
        cudaGetLastError();
        return splits;
    }
    for (uint32_t c = splits; c > splits / 2; --c) {
        const bool alone = slots_shared == 0 || ctas * c <= (uint64_t) sm_count / 2;
        const uint32_t slots = alone ? slots_alone : slots_shared;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned) (ctas * c));
        cfg.blockDim = dim3(kFusedThreads);
        cfg.dynamicSmemBytes = fused_smem_bytes(dhb, slots);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = c, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr, cfg.numAttrs = 1;
        int active = 0;
        if (cudaOccupancyMaxActiveClusters(&active, kernel, &cfg) != cudaSuccess) {
            cudaGetLastError();
            return splits;
        }
        if ((uint64_t) active >= ctas) return c;
    }
    return splits;
}

AttnFused *attn_fused_create(infiniopHandle_t handle, const AttnPrefillShape &s) {
    auto *h = reinterpret_cast<Handle *>(handle);
    // head sizes that are whole 16-byte vectors, up to 256: the TMA boxes are 64 elements wide and read what lies
    // beyond the head size as zeros, which changes neither q k^T nor the first dh columns of P v
    if (s.dh % 8 != 0 || s.dh == 0 || s.dh > 256) return nullptr;
    if (s.seq == 0 || s.total < s.seq || s.group == 0 || s.nh % s.group != 0) return nullptr;
    // TMA: strides in bytes are multiples of 16 and positive, rows do not overlap
    for (int64_t st : {s.q_s0, s.q_s1, s.kc_s0, s.kc_s1, s.vc_s0, s.vc_s1}) {
        if (st <= 0 || st % 8 != 0 || st >= ((int64_t) 1 << 38)) return nullptr;
    }
    if (s.q_s1 < (int64_t) s.dh || s.kc_s1 < (int64_t) s.dh || s.vc_s1 < (int64_t) s.dh) return nullptr;
    const uint32_t dhb = (s.dh + 63) / 64;
    uint32_t pack, tok;
    uint64_t blocks;
    fused_blocks(s, pack, tok, blocks);
    const uint64_t tiles_m = (s.seq + tok - 1) / tok;
    if (blocks > 0x7FFFFFFull) return nullptr;
    // A grid that leaves every CTA an SM of its own gets the whole shared memory for its ring of k / v tiles (the
    // loads of up to 11 tiles in flight hide the latency one CTA sees); otherwise two CTAs share an SM and each
    // takes half (4 tiles at dh 128), less the kilobyte the system keeps per CTA.
    int sm_bytes = 0;
    if (cudaDeviceGetAttribute(&sm_bytes, cudaDevAttrMaxSharedMemoryPerMultiprocessor, h->device_id) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    const uint32_t slots_alone = fused_slots(dhb, (size_t) h->max_smem_optin);
    const uint32_t slots_shared = fused_slots(dhb, (size_t) sm_bytes / 2 - 1024);
    const uint32_t splits = attn_fused_splits(s, h->sm_count, h->device_id);
    // (clusters: only while half the SMs suffice.  A cluster must find all its SMs in one GPC, and 16 clusters of
    // 8 CTAs with an SM each did not fit the GPCs at once: 86 us against 47 us with two CTAs per SM)
    // (head sizes beyond 128 take all of an SM's tensor memory and most of its shared memory: always alone)
    const bool alone = slots_shared == 0 || blocks * splits <= (uint64_t) h->sm_count / (splits > 1 ? 2 : 1);
    const uint32_t slots = alone ? slots_alone : slots_shared;
    if (slots == 0 || slots_alone == 0) return nullptr;
    const size_t smem = fused_smem_bytes(dhb, slots);
    FusedKernel kernel = fused_kernel(dhb);
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) fused_smem_bytes(dhb, slots_alone)) != cudaSuccess ||
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    auto *f = new (std::nothrow) AttnFused{};
    if (f == nullptr) return nullptr;
    f->device_id = h->device_id;
    f->shape = s;
    f->dhb = dhb, f->tiles_m = (uint32_t) tiles_m, f->slots = slots, f->splits = splits, f->smem_bytes = smem;
    f->pack = pack, f->tok = tok;
    // the encoder checks extents and strides, not the memory: a trial with a placeholder address tells now whether
    // these layouts can be described, so that the caller can keep its other path
    const void *probe = reinterpret_cast<const void *>((uintptr_t) 1 << 20);
    if (!encode_maps(f, probe, probe, probe)) {
        delete f;
        return nullptr;
    }
    return f;
}

infiniopStatus_t attn_fused_run(AttnFused *f, void *out, const void *q, const void *k_cache, const void *v_cache,
                                cudaStream_t st) {
    const AttnPrefillShape &s = f->shape;
    CUtensorMap mq, mk, mv;
    {
        std::lock_guard<std::mutex> lock(f->mu);
        if (!f->valid || f->q_ptr != q || f->k_ptr != k_cache || f->v_ptr != v_cache) {
            if (!encode_maps(f, q, k_cache, v_cache)) {
                f->valid = false;
                return STATUS_EXECUTION_FAILED;
            }
            f->valid = true, f->q_ptr = q, f->k_ptr = k_cache, f->v_ptr = v_cache;
        }
        mq = f->map_q, mk = f->map_k, mv = f->map_v;
    }
    FusedParams p{};
    p.nh = s.nh, p.group = s.group, p.seq = s.seq, p.total = s.total, p.tiles_m = f->tiles_m, p.slots = f->slots;
    p.dh = s.dh;
    p.splits = f->splits, p.pack = f->pack, p.tok = f->tok;
    p.alpha = (float) (1.0 / sqrt((double) s.dh));// `float qk_alpha = 1 / sqrt(head_dim)`, operator.cc:136
    p.out = reinterpret_cast<uint16_t *>(out);
    const uint32_t grid = f->tiles_m * (f->pack > 1 ? s.nh / s.group : s.nh) * f->splits;
    FusedKernel kernel = fused_kernel(f->dhb);
    // Programmatic dependent launch behind the cache append: the CTAs take their places, set up barriers and tensor
    // memory and load q while the append still runs; the loading lane waits for it before the first k tile.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = f->smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = f->splits, attr[1].val.clusterDim.y = 1, attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = f->splits > 1 ? 2 : 1;
    if (cudaLaunchKernelEx(&cfg, kernel, mq, mk, mv, p) != cudaSuccess) {
        cudaGetLastError();
        return STATUS_EXECUTION_FAILED;
    }
    return check_launch("attention (fused, several new tokens)");
}

void attn_fused_destroy(AttnFused *f) { delete f; }

#ifdef B200_ATTN_FUSED_TRACE
extern "C" __attribute__((visibility("default"))) int infiniopDebugAttnTrace(unsigned long long *out16, int reset) {
    if (cudaMemcpyFromSymbol(out16, g_attn_trace, 16 * sizeof(unsigned long long)) != cudaSuccess) return 1;
    if (reset) {
        unsigned long long zero[16] = {};
        if (cudaMemcpyToSymbol(g_attn_trace, zero, sizeof(zero)) != cudaSuccess) return 1;
    }
    return 0;
}
#endif

unsigned long long attn_fused_timeouts_read() {
    unsigned long long v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_tc_gemm_timeouts, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return ~0ull;
    }
    return v;
}

}// namespace b200
