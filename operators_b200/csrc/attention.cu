// Attention over a KV cache: k, v[n_kv_head, seq, dh] are written to the caches
// [n_kv_head, buf_len, dh] at rows pos .. pos+seq, then
//   out[i, head, :] = softmax_j(q[head, i, :] . K[kv, j, :] / sqrt(dh)) . V[kv, j, :],  j <= pos + i,
// with kv = head / (n_q_head / n_kv_head).
//
// Replaces the composite of reference src/ops/attention/operator.cc:30-305 (two
// rearranges into the caches, a rearrange of q, matmul, causal softmax, matmul,
// rearrange of the result; the nv-gpu matmuls are cuBLAS calls,
// src/ops/matmul/cuda/matmul_cuda.cu:8-77) behind include/ops/attention/attention.h.
// Arithmetic follows the CPU backend, roundings included: the scaled score is
// truncated to fp16 as the first matmul stores it (matmul_cpu.cc:63-65), the
// probability exp(s - max) / sum is truncated to fp16 as the softmax stores it
// (causal_softmax_cpu.cc:76-79) with exact zeros behind the mask, the output
// is truncated once more.  Only the grouping of the three fp32 sums differs
// (q.k, the softmax denominator, p.v), so `out` agrees with the CPU composite
// to a unit in the last place of fp16, not bit for bit.  The caches are byte-exact.
//
// Built for decoding, where the work is one read of the K and V rows of each kv
// head (HBM-bound: 4 * dh bytes per cached token and kv head).  kv_append_kernel
// copies the new rows into both caches; for a single new token the first of
// the other two kernels does that itself and there are two launches.  In these a
// CTA takes one kv head, up to 8 query rows that share it (the heads of its
// group x tokens) and one chunk of the cached tokens, so K and V are each read
// once however many q heads share them:
//  * attention_scores_kernel: the chunk's scores (to the workspace, fp16) with
//    their maximum and exp-sum.
//  * attention_values_kernel: every CTA merges the chunks' maxima and exp-sums
//    into its rows' maximum and denominator, forms the probabilities of its
//    chunk from the scores and writes the chunk's p . v to the workspace; the
//    CTA that arrives last for a (kv head, row tile) adds the chunks up and
//    writes `out`.
// Nothing waits on another CTA.  The scores cross the workspace because the
// reference's truncation of p needs the denominator of the whole row first;
// they are rows x tokens x 2 bytes against tokens x dh x 4 bytes of K and V.
// Prefill (many query rows) runs through the same kernels one row tile at a
// time, re-reading K and V per tile from L2: correct, not tuned; a tensor-core
// kernel is the next step for it.
#include "attention_prefill.cuh"
#include "common.cuh"

#include <cmath>
#include <cstdlib>
#include <new>

using namespace b200;

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxRows = 8;       // query rows per CTA
constexpr int kMaxChunk = 2048;   // cached tokens per CTA: their scores live in shared memory
constexpr int kMaxHeadDim = 256;
constexpr int kUnroll = 4;        // 128-bit loads in flight per thread
// Several new tokens, one kernel or three launches (microseconds, fitted to measurements at 32 q / 8 kv heads, dh
// 128): a CTA of the one-kernel form walks its tiles of 64 cached tokens alone, 1.64 us per tile (a cluster of up
// to 8 CTAs shares the tiles of a block of query rows when there are few blocks); the three launches cost 50 us
// plus 6 ps per score.  Grids that fill the GPU always take the one kernel (4096 new tokens: 0.28 ms against 1.70 ms).
constexpr double kFusedUsPerTile = 1.64, kFusedUsFixed = 8.0, kThreeUsFixed = 50.0, kThreeUsPerScore = 6e-6;

struct AttnDesc {
    Device device;
    int device_id;
    int sm_count;
    uint32_t nh, nkvh, group, seq, dh, pos, total;
    int64_t q_s0, q_s1, k_s0, k_s1, v_s0, v_s1, kc_s0, kc_s1, vc_s0, vc_s1;
    uint32_t rt, row_tiles, splits, chunk, tpk;
    bool strides_vec;             // every stride a multiple of 8 elements and dh % 8 == 0
    uint32_t score_pitch;         // splits * chunk: tokens per score row in the workspace
    uint64_t ws_ml, ws_acc, ws_scores, ws_bytes;// workspace: counters at 0, then the parts named here
    AttnPrefill *prefill;         // tensor-core path for calls with several new tokens (three launches), or null
    AttnFused *fused;             // the same in one kernel, or null
    uint64_t prefill_ws_bytes;
};

struct AttnArgs {
    uint16_t *out;
    const uint16_t *q, *k, *v;
    uint16_t *kc, *vc;
    uint32_t *counters;
    float2 *ml;   // per (kv head, tile, chunk, row): maximum and exp-sum of the chunk
    float *acc;   // per (kv head, tile, chunk, row): p . v of the chunk
    uint16_t *scores;
    uint32_t nh, nkvh, group, seq, dh, pos, total;
    int64_t q_s0, q_s1, k_s0, k_s1, v_s0, v_s1, kc_s0, kc_s1, vc_s0, vc_s1;
    uint32_t row_tiles, splits, chunk, score_pitch;
    uint32_t append_here;// one new token: the first of the two kernels writes its cache rows itself
    float alpha;
};

// Eight halves of a row starting at element 8 * sub; elements past `dh` read as zero.
template<bool VEC>
__device__ __forceinline__ uint4 load8(const uint16_t *row, uint32_t sub, uint32_t dh) {
    if (VEC) return ld_stream(row + sub * 8);
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const uint32_t c = sub * 8 + 2 * e;
        const uint32_t lo = c < dh ? row[c] : 0u, hi = c + 1 < dh ? row[c + 1] : 0u;
        w[e] = lo | (hi << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void unpack8(uint4 v, float (&f)[8]) {
    const uint32_t *p = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 t = unpack2(p[e]);
        f[2 * e] = t.x;
        f[2 * e + 1] = t.y;
    }
}

// k, v rows -> cache rows pos .. pos+seq of both caches; block 0 also clears the counters by which the
// last kernel finds the CTA that arrives last.
template<bool VEC>
__global__ void __launch_bounds__(kThreads) kv_append_kernel(AttnArgs a, uint32_t n_counters) {
    // a kernel launched behind this one as a programmatic dependent (the one-kernel attention form) may set itself
    // up meanwhile; it waits (griddepcontrol.wait) before it reads the caches
    asm volatile("griddepcontrol.launch_dependents;");
    if (blockIdx.x == 0) {
        for (uint32_t i = threadIdx.x; i < n_counters; i += kThreads) a.counters[i] = 0;
    }
    const uint32_t upr = VEC ? a.dh / 8 : a.dh;// units per row
    const uint64_t per_tensor = (uint64_t) a.nkvh * a.seq * upr;
    for (uint64_t idx = (uint64_t) blockIdx.x * kThreads + threadIdx.x; idx < 2 * per_tensor;
         idx += (uint64_t) gridDim.x * kThreads) {
        const bool is_v = idx >= per_tensor;
        uint64_t rem = is_v ? idx - per_tensor : idx;
        const uint32_t c = (uint32_t) (rem % upr);
        rem /= upr;
        const uint32_t i = (uint32_t) (rem % a.seq), h = (uint32_t) (rem / a.seq);
        const uint16_t *src = is_v ? a.v + (int64_t) h * a.v_s0 + (int64_t) i * a.v_s1
                                   : a.k + (int64_t) h * a.k_s0 + (int64_t) i * a.k_s1;
        uint16_t *dst = is_v ? a.vc + (int64_t) h * a.vc_s0 + (int64_t) (a.pos + i) * a.vc_s1
                             : a.kc + (int64_t) h * a.kc_s0 + (int64_t) (a.pos + i) * a.kc_s1;
        if (VEC) *reinterpret_cast<uint4 *>(dst + c * 8) = *reinterpret_cast<const uint4 *>(src + c * 8);
        else dst[c] = src[c];
    }
}

// Sum of v[r] over the TPK lanes of a key group, for all RT rows at once: while more than one row is left
// the two halves of the group exchange half of the rows each (a reduce-scatter), then single rows are
// summed both ways.  Afterwards this lane holds the complete sums of rows row_base .. row_base + kept
// (kept = max(1, RT / TPK)) in v[0 .. kept); `writer` is false on lanes that hold a duplicate.
template<int RT, int TPK>
__device__ __forceinline__ void group_sum(float (&v)[RT], uint32_t sub, int &row_base, bool &writer) {
    int n = RT;
    row_base = 0;
    writer = true;
#pragma unroll
    for (int off = TPK / 2; off >= 1; off >>= 1) {
        const bool upper = (sub & off) != 0;
        if (n > 1) {
            n >>= 1;
#pragma unroll
            for (int k = 0; k < RT / 2; ++k) {
                if (k < n) {
                    const float send = upper ? v[k] : v[k + n];
                    const float keep = upper ? v[k + n] : v[k];
                    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            if (upper) row_base += n;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
            if (upper) writer = false;
        }
    }
}

// What a CTA of either kernel works on: kv head, tile of query rows, chunk of cached tokens.
template<int RT>
struct Work {
    uint32_t split, h, tile, rows_total, c0, n;// n: tokens of the chunk that at least one row of the tile sees
    __device__ __forceinline__ Work(const AttnArgs &a) {
        split = blockIdx.x, h = blockIdx.y, tile = blockIdx.z;
        rows_total = a.group * a.seq;
        // row = g * seq + i of this kv head (the order the reference stacks the q heads of a kv head in); the tile's
        // last row sees the most tokens
        uint32_t top = tile * RT + RT - 1;
        if (top >= rows_total) top = rows_total - 1;
        int tile_last = -1;
        for (uint32_t row = tile * RT; row <= top; ++row) {
            const int lim = limit(a, row);
            tile_last = lim > tile_last ? lim : tile_last;
        }
        c0 = split * a.chunk;
        uint32_t c1 = c0 + a.chunk < a.total ? c0 + a.chunk : a.total;
        if ((int) c1 > tile_last + 1) c1 = (uint32_t) (tile_last + 1);
        n = c1 > c0 ? c1 - c0 : 0;
    }
    // last cached token the row sees (pos + i), -1 for rows past the end
    __device__ __forceinline__ int limit(const AttnArgs &a, uint32_t row) const {
        if (row >= rows_total) return -1;
        return (int) (a.pos + (row - (row / a.seq) * a.seq));
    }
    __device__ __forceinline__ uint64_t slot(const AttnArgs &a) const {// index of this CTA's first row among the partials
        return ((uint64_t) (h * a.row_tiles + tile) * a.splits + split) * RT;
    }
    __device__ __forceinline__ uint64_t first_slot(const AttnArgs &a) const {
        return (uint64_t) (h * a.row_tiles + tile) * a.splits * RT;
    }
    // fp16 scores of (row r of the tile, token j of the chunk) in the workspace
    __device__ __forceinline__ uint64_t score_at(const AttnArgs &a, uint32_t r, uint32_t j) const {
        return ((uint64_t) (h * a.row_tiles + tile) * RT + r) * a.score_pitch + c0 + j;
    }
};

// True in exactly one CTA of those that share a counter: the one that arrives last.  Everything the others
// wrote before arriving is visible to it afterwards.
__device__ __forceinline__ bool arrive_last(uint32_t *counter, uint32_t expected, int *flag) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *flag = atomicAdd(counter, 1u) == expected - 1;
    __syncthreads();
    const bool last = *flag != 0;
    if (last) __threadfence();
    return last;
}

// Decoding one token (seq == 1) does without the launch of kv_append_kernel: every CTA of the first kernel whose
// chunk holds cache row `pos` copies the token's k and v rows there before it reads the chunk (CTAs that share the
// chunk write the same bytes), and the CTAs of chunk 0 clear the counters of the second kernel.
template<bool VEC>
__device__ __forceinline__ void append_one_token(const AttnArgs &a, uint32_t h, uint32_t tile, uint32_t split) {
    if (!a.append_here) return;
    if (split == 0 && threadIdx.x == 0) a.counters[h * a.row_tiles + tile] = 0;
    const uint32_t c0 = split * a.chunk;
    if (a.pos < c0 || a.pos >= c0 + a.chunk) return;// the same answer in every thread of the CTA
    const uint32_t upr = VEC ? a.dh / 8 : a.dh;
    for (uint32_t u = threadIdx.x; u < 2 * upr; u += kThreads) {
        const bool is_v = u >= upr;
        const uint32_t c = is_v ? u - upr : u;
        const uint16_t *src = is_v ? a.v + (int64_t) h * a.v_s0 : a.k + (int64_t) h * a.k_s0;
        uint16_t *dst = is_v ? a.vc + (int64_t) h * a.vc_s0 + (int64_t) a.pos * a.vc_s1
                             : a.kc + (int64_t) h * a.kc_s0 + (int64_t) a.pos * a.kc_s1;
        if (VEC) *reinterpret_cast<uint4 *>(dst + c * 8) = *reinterpret_cast<const uint4 *>(src + c * 8);
        else dst[c] = src[c];
    }
    __syncthreads();
}

// After the chunk's scores stand in shared memory ([RT][pitch] floats): scores to the workspace with the chunk's
// row maxima and exp-sums.
template<int RT>
__device__ __forceinline__ void scores_epilogue(const AttnArgs &a, const Work<RT> &w, const float *smem, uint32_t pitch) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // per row: scores to the workspace, maximum and sum of exp(s - maximum) over the chunk; kWarps / RT warps share a row
    constexpr uint32_t WPR = kWarps / RT;
    __shared__ float part[2][kWarps];
    const uint32_t r = warp / WPR, seg = warp % WPR;
    const float *srow = smem + r * pitch;
    float m = -INFINITY;
    for (uint32_t j = seg * 32 + lane; j < w.n; j += WPR * 32) {
        const float sc = srow[j];
        m = fmaxf(m, sc);
        a.scores[w.score_at(a, r, j)] = __half_as_ushort(__float2half_rz(sc));// exact: an fp16 value or -inf
    }
    m = warp_max(m);
    if (lane == 0) part[0][warp] = m;
    __syncthreads();
    m = -INFINITY;
#pragma unroll
    for (uint32_t k = 0; k < WPR; ++k) m = fmaxf(m, part[0][r * WPR + k]);
    float l = 0.f;
    if (m > -INFINITY) {
        // base-2 exponential on the special-function unit (2^-22 relative): the sum only serves as the denominator
        for (uint32_t j = seg * 32 + lane; j < w.n; j += WPR * 32) l += fast_exp2((srow[j] - m) * 1.4426950408889634f);
    }
    l = warp_sum(l);
    if (lane == 0) part[1][warp] = l;
    __syncthreads();
    if (seg == 0 && lane == 0) {
        float total = 0.f;
#pragma unroll
        for (uint32_t k = 0; k < WPR; ++k) total += part[1][r * WPR + k];
        __stcg(a.ml + w.slot(a) + r, make_float2(m, total));
    }

}

// Maximum and denominator of row r of the tile over all chunks, from the chunks' (maximum, exp-sum) pairs the
// first kernel left; called by a whole warp.  Every CTA of the second kernel merges them for itself (a few
// dozen pairs from L2), which spares the first kernel a fence, a counter and a last-CTA pass.
template<int RT>
__device__ __forceinline__ float2 row_stat(const AttnArgs &a, const Work<RT> &w, uint32_t r) {
    const uint32_t lane = threadIdx.x & 31;
    const float2 *ml = a.ml + w.first_slot(a) + r;
    if (a.splits <= 32) {// one pair per lane: a single trip to memory
        const float2 part = lane < a.splits ? ml[(uint64_t) lane * RT] : make_float2(-INFINITY, 0.f);
        const float top = warp_max(part.x);
        return make_float2(top, warp_sum(part.x > -INFINITY ? part.y * expf(part.x - top) : 0.f));
    }
    float big = -INFINITY;
    for (uint32_t s = lane; s < a.splits; s += 32) big = fmaxf(big, ml[(uint64_t) s * RT].x);
    big = warp_max(big);
    float denom = 0.f;
    for (uint32_t s = lane; s < a.splits; s += 32) {
        const float2 part = ml[(uint64_t) s * RT];
        if (part.x > -INFINITY) denom = fmaf(part.y, expf(part.x - big), denom);
    }
    return make_float2(big, warp_sum(denom));
}

// ---- first kernel: scores = trunc16(alpha * q . k) of the chunk, row statistics ----------------------------
template<int RT, int TPK, bool VEC>
__global__ void __launch_bounds__(kThreads, 2) attention_scores_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float smem[];// scores [RT][chunk + 1]
    __shared__ int row_limit[RT];// last token each row of the tile sees
    constexpr int KPI = kThreads / TPK;// keys per iteration of the CTA
    constexpr int KEPT = RT / TPK > 1 ? RT / TPK : 1;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sub = tid % TPK, kg = tid / TPK;
    const bool col_live = sub * 8 < a.dh;
    const uint32_t pitch = a.chunk + 1;
    const Work<RT> w(a);
    append_one_token<VEC>(a, w.h, w.tile, w.split);

    float qf[RT][8];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const uint32_t row = w.tile * RT + r;
#pragma unroll
        for (int e = 0; e < 8; ++e) qf[r][e] = 0.f;
        if (row < w.rows_total && col_live) {
            const uint32_t g = row / a.seq, i = row - g * a.seq;
            const uint16_t *qr = a.q + (int64_t) (w.h * a.group + g) * a.q_s0 + (int64_t) i * a.q_s1;
            unpack8(load8<VEC>(qr, sub, a.dh), qf[r]);
        }
    }

    if (tid < RT) row_limit[tid] = w.limit(a, w.tile * RT + tid);
    __syncthreads();

    const uint16_t *kbase = a.kc + (int64_t) w.h * a.kc_s0 + (int64_t) w.c0 * a.kc_s1;
    // the loop bounds are the same for every thread (the sums below use warp shuffles); threads whose token
    // lies past the end work on zeros and write nothing
    for (uint32_t b = 0; b < w.n; b += KPI * kUnroll) {
        uint4 kv[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t j = b + u * KPI + kg;
            kv[u] = make_uint4(0, 0, 0, 0);
            if (j < w.n && col_live) kv[u] = load8<VEC>(kbase + (int64_t) j * a.kc_s1, sub, a.dh);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (b + u * KPI >= w.n) break;
            const uint32_t j = b + u * KPI + kg;
            float kf[8], dot[RT];
            unpack8(kv[u], kf);
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) s = fmaf(qf[r][e], kf[e], s);
                dot[r] = s;
            }
            int row_base;
            bool writer;
            group_sum<RT, TPK>(dot, sub, row_base, writer);
            if (writer && j < w.n) {
#pragma unroll
                for (int t = 0; t < KEPT; ++t) {
                    const int r = row_base + t;
                    float s = f16_to_f32(f32_to_f16_ref(__fmul_rn(a.alpha, dot[t])));// as the first matmul stores it
                    if ((int) (w.c0 + j) > row_limit[r]) s = -INFINITY;
                    smem[r * pitch + j] = s;
                }
            }
        }
    }
    __syncthreads();

    scores_epilogue<RT>(a, w, smem, pitch);
}

// After every warp's partial outputs stand in shared memory ([kWarps][RT][DHP] floats): their sum to the
// workspace, and in the CTA that arrives last the sum over the chunks to `out`.
template<int RT, int DHP>
__device__ __forceinline__ void values_epilogue(const AttnArgs &a, const Work<RT> &w, const float *smem, int *flag_ptr) {
    const uint32_t tid = threadIdx.x;
    const uint64_t slot = w.slot(a);
    for (uint32_t o = tid; o < RT * DHP; o += kThreads) {
        const uint32_t r = o / DHP, d = o - r * DHP;
        if (d < a.dh) {
            float s = 0.f;
#pragma unroll
            for (int wp = 0; wp < kWarps; ++wp) s += smem[(wp * RT + r) * DHP + d];
            __stcg(a.acc + (slot + r) * a.dh + d, s);
        }
    }

    // the last CTA of this (kv head, tile) adds the chunks up, first chunk first
    if (!arrive_last(a.counters + w.h * a.row_tiles + w.tile, a.splits, flag_ptr)) return;
    const uint64_t first = w.first_slot(a);
    for (uint32_t o = tid; o < RT * a.dh; o += kThreads) {
        const uint32_t r = o / a.dh, d = o - r * a.dh;
        const uint32_t row = w.tile * RT + r;
        if (row >= w.rows_total) continue;
        float sum = 0.f;
        for (uint32_t s = 0; s < a.splits; ++s) sum += __ldcg(a.acc + (first + (uint64_t) s * RT + r) * a.dh + d);
        const uint32_t g = row / a.seq, i = row - g * a.seq;
        a.out[((uint64_t) i * a.nh + w.h * a.group + g) * a.dh + d] = f32_to_f16_ref(sum);
    }
}

// ---- second kernel: p = trunc16(exp(s - max) / sum) as the softmax stores it, out = p . v -------------------
template<int RT, int TPK, bool VEC>
__global__ void __launch_bounds__(kThreads, 2) attention_values_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float smem[];// probabilities [RT][chunk + 1], later the per-warp outputs
    __shared__ int flag;
    constexpr int KPI = kThreads / TPK;
    constexpr int DHP = TPK * 8;// head dimension rounded up to the group's width
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sub = tid % TPK, kg = tid / TPK;
    const bool col_live = sub * 8 < a.dh;
    const uint32_t pitch = a.chunk + 1;
    const Work<RT> w(a);

    for (uint32_t r = warp; r < RT; r += kWarps) {
        const float2 st = row_stat<RT>(a, w, r);
        for (uint32_t j = lane; j < w.n; j += 32) {
            const float s = f16_to_f32(a.scores[w.score_at(a, r, j)]);
            float p = 0.f;// masked entries are exact zeros (causal_softmax_cpu.cc:68)
            if (s > -INFINITY) p = f16_to_f32(f32_to_f16_ref(__fdiv_rn(expf(s - st.x), st.y)));
            smem[r * pitch + j] = p;
        }
    }
    __syncthreads();

    float acc[RT][8];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[r][e] = 0.f;
    }
    const uint16_t *vbase = a.vc + (int64_t) w.h * a.vc_s0 + (int64_t) w.c0 * a.vc_s1;
    for (uint32_t j0 = kg; j0 < w.n; j0 += KPI * kUnroll) {
        uint4 vv[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t j = j0 + u * KPI;
            vv[u] = make_uint4(0, 0, 0, 0);
            if (j < w.n && col_live) vv[u] = load8<VEC>(vbase + (int64_t) j * a.vc_s1, sub, a.dh);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t j = j0 + u * KPI;
            if (j < w.n) {
                float vf[8];
                unpack8(vv[u], vf);
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    const float p = smem[r * pitch + j];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[r][e] = fmaf(p, vf[e], acc[r][e]);
                }
            }
        }
    }
    // key groups of one warp first (shuffles), then the warps through shared memory
#pragma unroll
    for (int off = TPK; off < 32; off <<= 1) {
#pragma unroll
        for (int r = 0; r < RT; ++r) {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[r][e] += __shfl_xor_sync(0xffffffffu, acc[r][e], off);
        }
    }
    __syncthreads();// every thread is done with the probabilities
    if (lane < TPK) {
#pragma unroll
        for (int r = 0; r < RT; ++r) {
#pragma unroll
            for (int e = 0; e < 8; ++e) smem[(warp * RT + r) * DHP + sub * 8 + e] = acc[r][e];
        }
    }
    __syncthreads();
    values_epilogue<RT, DHP>(a, w, smem, &flag);
}

// ---- the same two kernels with the dot products on the tensor cores ------------------------------------------
// mma.sync m16n8k16 (fp16 operands, fp32 accumulation): the eight columns of the result are the tile's query
// rows, so a kv head's rows cost the same whether one or eight q heads share them, and a lane needs one
// instruction per 16 bytes of K or V instead of eight multiply-adds per query row.  Used for 16-byte aligned
// rows with dh <= 128; nothing here is a GEMM-sized contraction, the kernels stay bound by the reads of K and V.
//
// A lane always loads 16 contiguous bytes of a cache row: lane = 4 * (row in a group of 8) + c, bytes
// [32 dh-block + 8 c, +8) halves.  The contraction index of an mma is only a label, so for q . k the
// four 32-bit registers of such a load serve as the k-pairs of two mmas directly, with q loaded the same way.
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// transpose of the 8 x 8 matrix of 16-bit values a warp holds one 32-bit register each of
__device__ __forceinline__ uint32_t transpose8x8(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

// 16 cache rows (row0 + lane / 4 and eight further down) x NB blocks of 32 halves; rows >= n and columns >= dh read as zero
template<int NB>
__device__ __forceinline__ void load_rows16(uint4 (&lo)[NB], uint4 (&hi)[NB], const uint16_t *base, int64_t row_stride,
                                            uint32_t row0, uint32_t n, uint32_t dh, uint32_t lane) {
    const uint32_t j_lo = row0 + (lane >> 2), j_hi = j_lo + 8, c = lane & 3;
#pragma unroll
    for (int blk = 0; blk < NB; ++blk) {
        const uint32_t col = blk * 32 + c * 8;
        lo[blk] = make_uint4(0, 0, 0, 0);
        hi[blk] = make_uint4(0, 0, 0, 0);
        if (col < dh) {
            if (j_lo < n) lo[blk] = ld_stream(base + (int64_t) j_lo * row_stride + col);
            if (j_hi < n) hi[blk] = ld_stream(base + (int64_t) j_hi * row_stride + col);
        }
    }
}

template<int RT, int NB>
__global__ void __launch_bounds__(kThreads, 2) attention_scores_mma_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float smem[];// scores [RT][chunk + 1]
    __shared__ int row_limit[8];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t kr = lane >> 2, c = lane & 3;
    const uint32_t pitch = a.chunk + 1;
    const Work<RT> w(a);
    asm volatile("griddepcontrol.launch_dependents;");// the second kernel's CTAs may queue up behind this one's
    // behind a cache append (several new tokens) this kernel is itself launched as a programmatic dependent: its CTAs
    // are in place when the append ends; without one the wait returns at once
    asm volatile("griddepcontrol.wait;" ::: "memory");
    append_one_token<true>(a, w.h, w.tile, w.split);
    if (tid < 8) row_limit[tid] = tid < RT ? w.limit(a, w.tile * RT + tid) : -1;

    // operand B: query row kr of the tile (zeros past the tile's rows)
    uint4 qb[NB];
#pragma unroll
    for (int blk = 0; blk < NB; ++blk) qb[blk] = make_uint4(0, 0, 0, 0);
    {
        const uint32_t row = w.tile * RT + kr;
        if (kr < RT && row < w.rows_total) {
            const uint32_t g = row / a.seq, i = row - g * a.seq;
            const uint16_t *qr = a.q + (int64_t) (w.h * a.group + g) * a.q_s0 + (int64_t) i * a.q_s1;
#pragma unroll
            for (int blk = 0; blk < NB; ++blk) {
                const uint32_t col = blk * 32 + c * 8;
                if (col < a.dh) qb[blk] = __ldg(reinterpret_cast<const uint4 *>(qr + col));
            }
        }
    }
    __syncthreads();

    // a warp takes groups of 16 tokens; the next group's rows are in flight while this one is multiplied
    const uint16_t *kbase = a.kc + (int64_t) w.h * a.kc_s0 + (int64_t) w.c0 * a.kc_s1;
    const uint32_t groups = (w.n + 15) / 16;
    uint4 lo[NB], hi[NB], nlo[NB], nhi[NB];
    if (warp < groups) load_rows16<NB>(lo, hi, kbase, a.kc_s1, warp * 16, w.n, a.dh, lane);
    auto multiply = [&](const uint4 (&lo)[NB], const uint4 (&hi)[NB], uint32_t gi) {
        float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int blk = 0; blk < NB; ++blk) {
            mma16816(d, lo[blk].x, hi[blk].x, lo[blk].y, hi[blk].y, qb[blk].x, qb[blk].y);
            mma16816(d, lo[blk].z, hi[blk].z, lo[blk].w, hi[blk].w, qb[blk].z, qb[blk].w);
        }
        // d[0], d[1]: token gi * 16 + kr, rows 2c and 2c + 1; d[2], d[3]: eight tokens further down
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint32_t j = gi * 16 + kr + (v >= 2 ? 8 : 0), r = 2 * c + (v & 1);
            if (r < RT && j < w.n) {
                float sc = f16_to_f32(f32_to_f16_ref(__fmul_rn(a.alpha, d[v])));// as the first matmul stores it
                if ((int) (w.c0 + j) > row_limit[r]) sc = -INFINITY;
                smem[r * pitch + j] = sc;
            }
        }
    };
    // two sets of registers take turns: one is multiplied while the other one's rows are in flight
    for (uint32_t gi = warp; gi < groups; gi += 2 * kWarps) {
        if (gi + kWarps < groups) load_rows16<NB>(nlo, nhi, kbase, a.kc_s1, (gi + kWarps) * 16, w.n, a.dh, lane);
        multiply(lo, hi, gi);
        if (gi + kWarps >= groups) break;
        if (gi + 2 * kWarps < groups) load_rows16<NB>(lo, hi, kbase, a.kc_s1, (gi + 2 * kWarps) * 16, w.n, a.dh, lane);
        multiply(nlo, nhi, gi + kWarps);
    }
    __syncthreads();
    scores_epilogue<RT>(a, w, smem, pitch);
}

// out^T[d][row] = sum_j V[j][d] * p[row][j]: operand A is V transposed, 8 x 8 blocks at a time in registers;
// operand B are the fp16 probabilities from shared memory.  Register t of a lane's 16-byte load holds columns
// d = 32 blk + 8 (m / 2) + 2 t + m % 2 of the block's rows m after the transposition.
template<int RT, int NB>
__global__ void __launch_bounds__(kThreads, 2) attention_values_mma_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float smem[];// fp16 probabilities [RT][chunk + 8], later the per-warp outputs
    __shared__ int flag;
    constexpr int DHP = NB * 32;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t kr = lane >> 2, c = lane & 3;
    const uint32_t pitch16 = a.chunk + 8;// in halves; rows land 4 banks apart
    uint16_t *p16 = reinterpret_cast<uint16_t *>(smem);
    const Work<RT> w(a);
    const uint32_t groups = (w.n + 15) / 16;

    // the first rows of V are on their way while the probabilities are formed
    const uint16_t *vbase = a.vc + (int64_t) w.h * a.vc_s0 + (int64_t) w.c0 * a.vc_s1;
    uint4 lo[NB], hi[NB], nlo[NB], nhi[NB];
    // (not in the chunk whose newest row the first kernel itself writes)
    const bool early = !(a.append_here && a.pos >= w.c0 && a.pos < w.c0 + a.chunk);
    if (early && warp < groups) load_rows16<NB>(lo, hi, vbase, a.vc_s1, warp * 16, w.n, a.dh, lane);
    asm volatile("griddepcontrol.wait;" ::: "memory");// everything the first kernel wrote is visible from here on
    if (!early && warp < groups) load_rows16<NB>(lo, hi, vbase, a.vc_s1, warp * 16, w.n, a.dh, lane);

    // probabilities of the chunk: kWarps / RT warps per row, eight scores per lane and step
    {
        constexpr uint32_t WPR = kWarps / RT;
        const uint32_t r = warp / WPR, seg = warp % WPR;
        const uint16_t *srow = a.scores + w.score_at(a, r, 0);// 16-byte aligned: chunk and pitch are multiples of 64
        // the first scores are requested before the row's statistics are merged (both come from L2 or HBM)
        constexpr uint32_t kStep = WPR * 256, kAhead = 4;
        const uint32_t j0 = (seg * 32 + lane) * 8, lim = groups * 16;
        uint4 ahead[kAhead];
#pragma unroll
        for (uint32_t u = 0; u < kAhead; ++u) {
            ahead[u] = make_uint4(0, 0, 0, 0);
            if (j0 + u * kStep < lim) ahead[u] = __ldcs(reinterpret_cast<const uint4 *>(srow + j0 + u * kStep));
        }
        const float2 st = row_stat<RT>(a, w, r);
        // exp(s - max) / sum as 2^((s - max) log2 e) * (1 / sum): within 2^-21 of the quotient before the truncation
        const float inv_sum = __frcp_rn(st.y);
        auto emit = [&](uint4 raw, uint32_t j) {
            const uint16_t *sc16 = reinterpret_cast<const uint16_t *>(&raw);
            uint32_t packed[4];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                uint32_t bits = 0;// masked entries and the padding of the last group are exact zeros
                const float sc = f16_to_f32(sc16[e]);
                if (j + e < w.n && sc > -INFINITY) {
                    bits = f32_to_f16_ref(fast_exp2((sc - st.x) * 1.4426950408889634f) * inv_sum);
                }
                packed[e >> 1] = (e & 1) ? (packed[e >> 1] | (bits << 16)) : bits;
            }
            *reinterpret_cast<uint4 *>(p16 + r * pitch16 + j) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        };
#pragma unroll
        for (uint32_t u = 0; u < kAhead; ++u) {
            if (j0 + u * kStep < lim) emit(ahead[u], j0 + u * kStep);
        }
        for (uint32_t j = j0 + kAhead * kStep; j < lim; j += kStep) emit(__ldcs(reinterpret_cast<const uint4 *>(srow + j)), j);
    }
    __syncthreads();

    float acc[NB][2][4];
#pragma unroll
    for (int blk = 0; blk < NB; ++blk) {
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[blk][0][v] = acc[blk][1][v] = 0.f;
    }
    auto multiply = [&](const uint4 (&lo)[NB], const uint4 (&hi)[NB], uint32_t gi) {
        uint32_t b0 = 0, b1 = 0;// probabilities of row kr for tokens 2c, 2c+1 and eight further down
        if (kr < RT) {
            const uint16_t *pr = p16 + kr * pitch16 + gi * 16 + 2 * c;
            b0 = *reinterpret_cast<const uint32_t *>(pr);
            b1 = *reinterpret_cast<const uint32_t *>(pr + 8);
        }
#pragma unroll
        for (int blk = 0; blk < NB; ++blk) {
            mma16816(acc[blk][0], transpose8x8(lo[blk].x), transpose8x8(lo[blk].y), transpose8x8(hi[blk].x),
                     transpose8x8(hi[blk].y), b0, b1);
            mma16816(acc[blk][1], transpose8x8(lo[blk].z), transpose8x8(lo[blk].w), transpose8x8(hi[blk].z),
                     transpose8x8(hi[blk].w), b0, b1);
        }
    };
    for (uint32_t gi = warp; gi < groups; gi += 2 * kWarps) {// two sets of registers take turns, as in the first kernel
        if (gi + kWarps < groups) load_rows16<NB>(nlo, nhi, vbase, a.vc_s1, (gi + kWarps) * 16, w.n, a.dh, lane);
        multiply(lo, hi, gi);
        if (gi + kWarps >= groups) break;
        if (gi + 2 * kWarps < groups) load_rows16<NB>(lo, hi, vbase, a.vc_s1, (gi + 2 * kWarps) * 16, w.n, a.dh, lane);
        multiply(nlo, nhi, gi + kWarps);
    }
    __syncthreads();// every warp is done with the probabilities
#pragma unroll
    for (int blk = 0; blk < NB; ++blk) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint32_t d = blk * 32 + (kr >> 1) * 8 + 2 * (2 * u + (v >> 1)) + (kr & 1), r = 2 * c + (v & 1);
                if (r < RT) smem[(warp * RT + r) * DHP + d] = acc[blk][u][v];
            }
        }
    }
    __syncthreads();
    values_epilogue<RT, DHP>(a, w, smem, &flag);
}

template<int RT, int NB>
infiniopStatus_t launch_mma(const AttnDesc *d, const AttnArgs &args, cudaStream_t st) {
    constexpr int DHP = NB * 32;
    const size_t smem_scores = (size_t) RT * (d->chunk + 1) * sizeof(float);
    size_t smem_values = (size_t) RT * (d->chunk + 8) * sizeof(uint16_t);
    const size_t red = (size_t) kWarps * RT * DHP * sizeof(float);
    if (red > smem_values) smem_values = red;
    static thread_local int configured_dev = -1;
    if (configured_dev != d->device_id) {
        constexpr size_t most = (size_t) kMaxRows * (kMaxChunk + 1) * sizeof(float);
        if (cudaFuncSetAttribute(attention_scores_mma_kernel<RT, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int) most) != cudaSuccess ||
            cudaFuncSetAttribute(attention_values_mma_kernel<RT, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int) most) != cudaSuccess) {
            cudaGetLastError();
            return STATUS_EXECUTION_FAILED;
        }
        configured_dev = d->device_id;
    }
    const dim3 grid(d->splits, d->nkvh, d->row_tiles);
    if (args.append_here) {
        attention_scores_mma_kernel<RT, NB><<<grid, kThreads, smem_scores, st>>>(args);
    } else {// the append kernel runs ahead of this one
        cudaLaunchConfig_t first = {};
        first.gridDim = grid;
        first.blockDim = dim3(kThreads);
        first.dynamicSmemBytes = smem_scores;
        first.stream = st;
        cudaLaunchAttribute dep[1];
        dep[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        dep[0].val.programmaticStreamSerializationAllowed = 1;
        first.attrs = dep;
        first.numAttrs = 1;
        if (cudaLaunchKernelEx(&first, attention_scores_mma_kernel<RT, NB>, args) != cudaSuccess) {
            cudaGetLastError();
            return STATUS_EXECUTION_FAILED;
        }
    }
    const infiniopStatus_t status = check_launch("attention scores");
    if (status != STATUS_SUCCESS) return status;
    // Programmatic dependent launch: the CTAs of the second kernel may take their places while the last CTAs of the
    // first are still at work; they request their first rows of V and then wait (griddepcontrol.wait) until the
    // whole first kernel has finished and its scores are visible.  The first kernel releases them when it starts.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_values;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, attention_values_mma_kernel<RT, NB>, args) != cudaSuccess) {
        cudaGetLastError();
        return STATUS_EXECUTION_FAILED;
    }
    return check_launch("attention values");
}

template<int RT>
infiniopStatus_t launch_mma_blocks(const AttnDesc *d, const AttnArgs &args, cudaStream_t st) {
    if (d->dh <= 32) return launch_mma<RT, 1>(d, args, st);
    if (d->dh <= 64) return launch_mma<RT, 2>(d, args, st);
    return launch_mma<RT, 4>(d, args, st);
}

infiniopStatus_t launch_mma_rows(const AttnDesc *d, const AttnArgs &args, cudaStream_t st) {
    switch (d->rt) {
        case 1: return launch_mma_blocks<1>(d, args, st);
        case 2: return launch_mma_blocks<2>(d, args, st);
        case 4: return launch_mma_blocks<4>(d, args, st);
        default: return launch_mma_blocks<8>(d, args, st);
    }
}

template<int RT, int TPK, bool VEC>
infiniopStatus_t launch_split(const AttnDesc *d, const AttnArgs &args, cudaStream_t st) {
    constexpr int DHP = TPK * 8;
    const size_t smem_scores = (size_t) RT * (d->chunk + 1) * sizeof(float);
    size_t smem_values = smem_scores;
    const size_t red = (size_t) kWarps * RT * DHP * sizeof(float);
    if (red > smem_values) smem_values = red;
    static thread_local int configured_dev = -1;
    if (configured_dev != d->device_id) {
        constexpr size_t most = (size_t) kMaxRows * (kMaxChunk + 1) * sizeof(float);
        if (cudaFuncSetAttribute(attention_scores_kernel<RT, TPK, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int) most) != cudaSuccess ||
            cudaFuncSetAttribute(attention_values_kernel<RT, TPK, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int) most) != cudaSuccess) {
            cudaGetLastError();
            return STATUS_EXECUTION_FAILED;
        }
        configured_dev = d->device_id;
    }
    const dim3 grid(d->splits, d->nkvh, d->row_tiles);
    attention_scores_kernel<RT, TPK, VEC><<<grid, kThreads, smem_scores, st>>>(args);
    const infiniopStatus_t status = check_launch("attention scores");
    if (status != STATUS_SUCCESS) return status;
    attention_values_kernel<RT, TPK, VEC><<<grid, kThreads, smem_values, st>>>(args);
    return check_launch("attention values");
}

template<int RT, bool VEC>
infiniopStatus_t launch_tpk(const AttnDesc *d, const AttnArgs &args, cudaStream_t st) {
    switch (d->tpk) {
        case 1: return launch_split<RT, 1, VEC>(d, args, st);
        case 2: return launch_split<RT, 2, VEC>(d, args, st);
        case 4: return launch_split<RT, 4, VEC>(d, args, st);
        case 8: return launch_split<RT, 8, VEC>(d, args, st);
        case 16: return launch_split<RT, 16, VEC>(d, args, st);
        default: return launch_split<RT, 32, VEC>(d, args, st);
    }
}

template<bool VEC>
infiniopStatus_t launch_rows(const AttnDesc *d, const AttnArgs &args, cudaStream_t st) {
    switch (d->rt) {
        case 1: return launch_tpk<1, VEC>(d, args, st);
        case 2: return launch_tpk<2, VEC>(d, args, st);
        case 4: return launch_tpk<4, VEC>(d, args, st);
        default: return launch_tpk<8, VEC>(d, args, st);
    }
}

}// namespace

INFINIOP_API infiniopStatus_t infiniopCreateAttentionDescriptor(infiniopHandle_t handle,
                                                                infiniopAttentionDescriptor_t *desc_ptr,
                                                                infiniopTensorDescriptor_t out_desc,
                                                                infiniopTensorDescriptor_t q_desc,
                                                                infiniopTensorDescriptor_t k_desc,
                                                                infiniopTensorDescriptor_t v_desc,
                                                                infiniopTensorDescriptor_t k_cache_desc,
                                                                infiniopTensorDescriptor_t v_cache_desc, uint64_t pos) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    infiniopTensorDescriptor_t all[6] = {out_desc, q_desc, k_desc, v_desc, k_cache_desc, v_cache_desc};
    for (auto *t : all) {
        if (t == nullptr) return STATUS_BAD_PARAM;
    }
    // checks, order and codes of reference src/ops/attention/operator.cc:39-86
    for (auto *t : all) {
        if (t->ndim != 3) return STATUS_BAD_TENSOR_SHAPE;
    }
    if (out_desc->strides[2] != 1 || out_desc->strides[1] != (int64_t) out_desc->shape[2] ||
        out_desc->strides[0] != (int64_t) (out_desc->shape[1] * out_desc->shape[2])) {
        return STATUS_BAD_TENSOR_STRIDES;// out must be contiguous
    }
    for (int t = 1; t < 6; ++t) {
        if (all[t]->strides[2] != 1) return STATUS_BAD_TENSOR_STRIDES;
    }
    const uint64_t nh = q_desc->shape[0], seq = q_desc->shape[1], dh = q_desc->shape[2], nkvh = k_desc->shape[0];
    const uint64_t total = seq + pos;
    if (out_desc->shape[0] != seq || out_desc->shape[1] != nh || out_desc->shape[2] != dh) return STATUS_BAD_PARAM;
    if (k_desc->shape[1] != seq || k_desc->shape[2] != dh) return STATUS_BAD_PARAM;
    if (v_desc->shape[0] != nkvh || v_desc->shape[1] != seq || v_desc->shape[2] != dh) return STATUS_BAD_PARAM;
    if (k_cache_desc->shape[0] != nkvh || k_cache_desc->shape[1] < total || k_cache_desc->shape[2] != dh) return STATUS_BAD_PARAM;
    if (v_cache_desc->shape[0] != nkvh || v_cache_desc->shape[1] < total || v_cache_desc->shape[2] != dh) return STATUS_BAD_PARAM;
    if (nkvh == 0 || nh % nkvh != 0) return STATUS_BAD_PARAM;// the reference's dim_split of the q heads fails
    // fp16 only here (the reference's matmul also takes fp32, its causal softmax does not)
    for (auto *t : all) {
        if (!dt_eq(t->dt, F16)) return STATUS_BAD_TENSOR_DTYPE;
    }
    if (dh == 0 || dh > (uint64_t) kMaxHeadDim || total > 0x7FFFFFFFull || nh > 0xFFFFull || seq > 0xFFFFFFull ||
        nh / nkvh * seq > 0x7FFFFFFFull) {
        return STATUS_BAD_TENSOR_SHAPE;
    }

    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow) AttnDesc{};
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    d->device = DevNvGpu;
    d->device_id = h->device_id;
    d->sm_count = h->sm_count;
    d->nh = (uint32_t) nh, d->nkvh = (uint32_t) nkvh, d->group = (uint32_t) (nh / nkvh), d->seq = (uint32_t) seq;
    d->dh = (uint32_t) dh, d->pos = (uint32_t) pos, d->total = (uint32_t) total;
    d->q_s0 = q_desc->strides[0], d->q_s1 = q_desc->strides[1];
    d->k_s0 = k_desc->strides[0], d->k_s1 = k_desc->strides[1];
    d->v_s0 = v_desc->strides[0], d->v_s1 = v_desc->strides[1];
    d->kc_s0 = k_cache_desc->strides[0], d->kc_s1 = k_cache_desc->strides[1];
    d->vc_s0 = v_cache_desc->strides[0], d->vc_s1 = v_cache_desc->strides[1];
    const int64_t strides[10] = {d->q_s0, d->q_s1, d->k_s0, d->k_s1, d->v_s0, d->v_s1, d->kc_s0, d->kc_s1, d->vc_s0, d->vc_s1};
    d->strides_vec = dh % 8 == 0;
    for (int64_t s : strides) d->strides_vec = d->strides_vec && s % 8 == 0;

    // rows per CTA: all query rows of a kv head when there are at most 8 (decoding), tiles of 8 otherwise
    const uint64_t rows = (uint64_t) d->group * seq;
    d->rt = rows <= 1 ? 1 : rows <= 2 ? 2 : rows <= 4 ? 4 : 8;
    d->row_tiles = (uint32_t) ((rows + d->rt - 1) / d->rt);
    uint32_t tpk = 1;
    while (tpk * 8 < dh) tpk *= 2;
    d->tpk = tpk;
    if (d->row_tiles > 65535u || nkvh > 65535ull) {// grid dimensions y and z
        delete d;
        return STATUS_BAD_TENSOR_SHAPE;
    }
    // Chunks of the cached tokens, 64 .. kMaxChunk tokens each.  Two CTAs fit an SM and the kernels are fastest
    // when the grid is a whole number of such resident sets (a few CTAs beyond one would run alone at the end):
    // the smallest number of sets whose chunks stay within kMaxChunk.
    if (total > 0) {
        const uint64_t base = (uint64_t) nkvh * d->row_tiles;
        uint64_t per_set = 2ull * d->sm_count / base;
        if (per_set < 1) per_set = 1;
        const uint64_t least = (total + kMaxChunk - 1) / kMaxChunk, most = (total + 63) / 64;
        uint64_t splits = (least + per_set - 1) / per_set * per_set;
        if (splits > most) splits = most;
        const uint64_t chunk = ((total + splits - 1) / splits + 63) / 64 * 64;
        d->chunk = (uint32_t) chunk;
        d->splits = (uint32_t) ((total + chunk - 1) / chunk);
    } else {
        d->chunk = 64;
        d->splits = 1;
    }
    const uint64_t tiles = (uint64_t) nkvh * d->row_tiles, slots = tiles * d->splits * d->rt;
    auto pad = [](uint64_t bytes) { return (bytes + 255) / 256 * 256; };
    d->score_pitch = d->splits * d->chunk;
    d->ws_ml = pad(tiles * sizeof(uint32_t));// one counter per tile
    d->ws_acc = d->ws_ml + pad(slots * sizeof(float2));
    d->ws_scores = d->ws_acc + pad(slots * dh * sizeof(float));
    d->ws_bytes = d->ws_scores + pad(tiles * d->rt * (uint64_t) d->score_pitch * sizeof(uint16_t));
    // several new tokens per q head: the products go to the tensor-core matmul (attention_prefill.cu)
    d->prefill = nullptr;
    d->prefill_ws_bytes = 0;
    // (measured, 32 q / 8 kv heads, dh 128: 8 new tokens over 4096 cached 46 us against 29 us for the row-tile kernels,
    // 16 tokens 48 against 40, 64 tokens over 8192 cached 146 against 191, 512 tokens from an empty cache 92 against 115)
    d->fused = nullptr;
    // (from 16 tokens when the q heads of a kv head can share a block of query rows: 16 tokens over 4096 cached run
    // faster there than on the row-tile kernels)
    if (seq >= (d->group > 1 ? 16u : 32u) && d->strides_vec && total > 0) {
        const AttnPrefillShape shape{d->nh, d->group, d->seq, d->dh, d->total, d->q_s0, d->q_s1, d->kc_s0, d->kc_s1, d->vc_s0, d->vc_s1};
        // One kernel that keeps the scores on chip (attention_fused.cu) unless the model says that its CTAs (per
        // 128 query rows of a head: one, or a cluster of up to 8 that splits the cached tokens) would walk their
        // tokens for longer than the three launches take, which spread the cached tokens over the whole GPU
        // (few heads and a very long cache).  The choice is made here because
        // the two paths need different workspaces; infiniopExtSelectKernel(attention, 3 / 4) forces either.
        const int choice = kernel_choice(kFamilyAttention);
        const uint64_t ctas = (uint64_t) ((seq + 127) / 128) * d->nh, kv_tiles = (total + 63) / 64;
        const uint32_t splits = attn_fused_splits(shape, d->sm_count, d->device_id);// CTAs of a cluster that share a block of query rows
        const double one_us = kFusedUsFixed + kFusedUsPerTile * (double) ((kv_tiles + splits - 1) / splits) + (splits > 1 ? 6.0 : 0.0);
        const double three_us = kThreeUsFixed + kThreeUsPerScore * (double) d->nh * (double) seq * (double) total;
        if (choice == 4 || (choice != 3 && (ctas > (uint64_t) d->sm_count || one_us < three_us))) {
            d->fused = attn_fused_create(handle, shape);
        }
        if (d->fused == nullptr) {
            d->prefill = attn_prefill_create(handle, shape, &d->prefill_ws_bytes);
            if (d->prefill != nullptr && d->prefill_ws_bytes > d->ws_bytes) d->ws_bytes = d->prefill_ws_bytes;
        }
    }
    *desc_ptr = reinterpret_cast<infiniopAttentionDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetAttentionWorkspaceSize(infiniopAttentionDescriptor_t desc, uint64_t *size) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = reinterpret_cast<AttnDesc *>(desc)->ws_bytes;
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopAttention(infiniopAttentionDescriptor_t desc, void *workspace,
                                                uint64_t workspace_size, void *out, void const *q, void const *k,
                                                void const *v, void *k_cache, void *v_cache, void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    auto *d = reinterpret_cast<AttnDesc *>(desc);
    if (workspace_size < d->ws_bytes || workspace == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;// operator.cc:264-266
    if (out == nullptr || q == nullptr || k == nullptr || v == nullptr || k_cache == nullptr || v_cache == nullptr) {
        return STATUS_BAD_PARAM;
    }
    if (d->seq == 0 || d->nh == 0) return STATUS_SUCCESS;
    if (!aligned16(workspace)) return STATUS_BAD_PARAM;
    DeviceGuard guard(d->device_id);
    auto st = reinterpret_cast<cudaStream_t>(stream);
    auto *ws = reinterpret_cast<uint8_t *>(workspace);
    AttnArgs a{};
    a.out = reinterpret_cast<uint16_t *>(out);
    a.q = reinterpret_cast<const uint16_t *>(q), a.k = reinterpret_cast<const uint16_t *>(k);
    a.v = reinterpret_cast<const uint16_t *>(v);
    a.kc = reinterpret_cast<uint16_t *>(k_cache), a.vc = reinterpret_cast<uint16_t *>(v_cache);
    a.counters = reinterpret_cast<uint32_t *>(ws);
    a.ml = reinterpret_cast<float2 *>(ws + d->ws_ml);
    a.acc = reinterpret_cast<float *>(ws + d->ws_acc);
    a.scores = reinterpret_cast<uint16_t *>(ws + d->ws_scores);
    a.nh = d->nh, a.nkvh = d->nkvh, a.group = d->group, a.seq = d->seq, a.dh = d->dh, a.pos = d->pos, a.total = d->total;
    a.q_s0 = d->q_s0, a.q_s1 = d->q_s1, a.k_s0 = d->k_s0, a.k_s1 = d->k_s1, a.v_s0 = d->v_s0, a.v_s1 = d->v_s1;
    a.kc_s0 = d->kc_s0, a.kc_s1 = d->kc_s1, a.vc_s0 = d->vc_s0, a.vc_s1 = d->vc_s1;
    a.row_tiles = d->row_tiles, a.splits = d->splits, a.chunk = d->chunk, a.score_pitch = d->score_pitch;
    a.alpha = (float) (1.0 / sqrt((double) d->dh));// `float qk_alpha = 1 / sqrt(head_dim)`, operator.cc:136

    const bool vec = d->strides_vec && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(k_cache) && aligned16(v_cache);
    const uint32_t n_counters = d->nkvh * d->row_tiles;
    const uint64_t units = 2ull * d->nkvh * d->seq * (vec ? d->dh / 8 : d->dh);
    uint64_t ctas = (units + kThreads - 1) / kThreads;
    const uint64_t cap = (uint64_t) d->sm_count * 8;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    a.append_here = d->seq == 1;
    if (!a.append_here) {
        if (vec) kv_append_kernel<true><<<(uint32_t) ctas, kThreads, 0, st>>>(a, n_counters);
        else kv_append_kernel<false><<<(uint32_t) ctas, kThreads, 0, st>>>(a, n_counters);
        const infiniopStatus_t status = check_launch("attention kv append");
        if (status != STATUS_SUCCESS) return status;
    }
    // several new tokens: one kernel, or scores, softmax and values as three tensor-core / streaming launches
    const int choice = kernel_choice(kFamilyAttention);
    if (d->fused != nullptr && vec && aligned16(out) && (choice == 0 || choice >= 3)) {
        return attn_fused_run(d->fused, out, q, k_cache, v_cache, st);
    }
    if (d->prefill != nullptr && vec && (choice == 0 || choice >= 3)) {
        return attn_prefill_run(d->prefill, workspace, out, q, k_cache, v_cache, st);
    }
    // the multiply-add kernels serve unaligned layouts and head sizes above 128 (and every layout when
    // infiniopExtSelectKernel asked for them)
    if (vec && d->dh <= 128 && kernel_choice(kFamilyAttention) != 1) return launch_mma_rows(d, a, st);
    return vec ? launch_rows<true>(d, a, st) : launch_rows<false>(d, a, st);
}

INFINIOP_API infiniopStatus_t infiniopDestroyAttentionDescriptor(infiniopAttentionDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    auto *d = reinterpret_cast<AttnDesc *>(desc);
    attn_prefill_destroy(d->prefill);
    attn_fused_destroy(d->fused);
    delete d;
    return STATUS_SUCCESS;
}
