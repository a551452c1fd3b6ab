// Long rows of RMSNorm and causal softmax staged in shared memory.
//
// The register-resident kernels load a row, reduce it, scale it and store it, a few rows per SM at a time; for rows of
// 32 Ki elements and more too few loads are in flight.  Here one persistent CTA per SM (or one cluster of 2 / 4 / 8
// CTAs for rows that do not fit one CTA's shared memory three times) keeps a ring of row buffers in shared memory:
// one thread requests whole rows with cp.async.bulk (TMA) two rows ahead, completion counted in bytes on an mbarrier;
// all threads reduce the row out of shared memory, scale it and store the results straight to global memory (128-bit
// streaming stores); the buffer is requested again for the row three ahead.  Loads of the next rows are therefore
// always in flight while a row is processed; what bounds the ring is the four CTA-wide barriers per row.  Measured on
// 256 MB of rows it beats the register kernels for RMSNorm rows of 32 Ki and 64 Ki elements (4.3 against 3.7 TB/s, 3.2
// against 2.8 TB/s) and nowhere for causal softmax, so RMSNorm takes it by itself in that range and softmax only
// when infiniopExtSelectKernel asks.  Cluster form: CTA r holds vectors [r * part, (r + 1) * part) of every row of
// its cluster, the partial maxima / sums meet over distributed shared memory (cluster_reduce), one cluster barrier
// closes a row.
//
// Every mbarrier wait is bounded.  A CTA whose wait runs out keeps walking its rows without touching them (so that
// it still meets its cluster at every barrier), counts itself in the file's timeout counter and leaves; the rows it
// skipped stay unwritten and infiniopExtDeviceTimeouts reports it.
#pragma once

#include "bulk_copy.cuh"
#include "common.cuh"

namespace b200 {
namespace ring {

using namespace bulk;

constexpr int kThreads = 1024;
constexpr int kStages = 3;
constexpr uint32_t kMaxPartBytes = 72 * 1024;// 3 stages of 72 KB = 216 KB

// per translation unit that includes this header
static __device__ unsigned int g_row_ring_timeouts = 0;

struct Plan {
    uint32_t cl;        // CTAs per row (1, 2, 4, 8)
    uint32_t part_vecs; // 128-bit vectors of a row per CTA (the last CTA of a cluster may hold fewer)
    uint32_t grid;      // CTAs in all
    size_t smem_bytes;
};

// Rows of `vecs` vectors; false when even eight CTAs cannot hold a row three times.
static inline bool make_plan(Plan &p, uint32_t vecs, uint64_t rows, int sm_count) {
    uint32_t cl = 1;
    while (cl <= 8 && (uint64_t) ((vecs + cl - 1) / cl) * 16 > kMaxPartBytes) cl *= 2;
    if (cl > 8) return false;
    p.cl = cl;
    p.part_vecs = (vecs + cl - 1) / cl;
    uint64_t clusters = (uint64_t) sm_count / cl;
    if (clusters > rows) clusters = rows;
    if (clusters < 1) clusters = 1;
    p.grid = (uint32_t) clusters * cl;
    p.smem_bytes = (size_t) kStages * p.part_vecs * 16;
    return true;
}

// The ring of one CTA: `issue(i)` is called by thread 0 with the index of the row (of this CTA's sequence) to request
// into stage i % kStages; it returns the bytes requested (0: nothing to load, the barrier is completed at once).
struct Ring {
    uint64_t *full;
    unsigned char *stages;
    uint32_t stage_bytes;
    __device__ __forceinline__ unsigned char *stage(uint32_t i) const { return stages + (size_t) (i % kStages) * stage_bytes; }
    __device__ __forceinline__ void request(uint32_t i, const void *src, uint32_t bytes) const {
        uint64_t *bar = &full[i % kStages];
        mbar_expect_tx(bar, bytes);// bytes may be 0: the arrival alone completes the phase
        if (bytes) bulk_load(stage(i), src, bytes, bar);
    }
    // all threads; false when the wait ran out
    __device__ __forceinline__ bool wait(uint32_t i, uint32_t polls) const {
        return mbar_wait_bounded(&full[i % kStages], (i / kStages) & 1u, polls);
    }
};

// ---------------------------------------------------------------- RMSNorm --
// SCALE(ss) -> the two-float scale; OUT(k, x_word, w...) are supplied by rms_norm.cu through these functors so that the
// arithmetic stays in one place.
template<int DT, bool W_F16, typename ScaleFn, typename ProdFn>
__device__ __forceinline__ void rms_norm_ring_body(uint16_t *y, const uint16_t *x, const void *w, uint64_t n, uint32_t vecs,
                                                   uint64_t d, int64_t stride_y, int64_t stride_x, float eps, Plan plan,
                                                   ScaleFn scale_of, ProdFn prod) {
    extern __shared__ __align__(128) unsigned char ring_smem[];
    __shared__ __align__(8) uint64_t full[kStages];
    __shared__ float red[32];
    __shared__ float part;
    __shared__ int s_fail;
    const uint32_t cl = plan.cl, rank = cl > 1 ? cluster_rank() : 0;
    const uint32_t clusters = gridDim.x / cl, me = blockIdx.x / cl;
    const uint32_t v0 = rank * plan.part_vecs;// this CTA's vectors of every row: [v0, v0 + nv)
    const uint32_t nv = v0 >= vecs ? 0u : (vecs - v0 < plan.part_vecs ? vecs - v0 : plan.part_vecs);
    const uint32_t cnt = me < n ? (uint32_t) ((n - me + clusters - 1) / clusters) : 0u;// rows of this cluster
    const Ring rg{full, ring_smem, plan.part_vecs * 16u};
    auto row_of = [&](uint32_t i) { return (uint64_t) me + (uint64_t) i * clusters; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (uint32_t i = 0; i < cnt && i < (uint32_t) kStages; ++i) {
            rg.request(i, x + (int64_t) row_of(i) * stride_x + (size_t) v0 * 8, nv * 16u);
        }
    }
    __syncthreads();
    uint32_t polls = kWaitPolls;
    for (uint32_t i = 0; i < cnt; ++i) {
        const bool arrived = rg.wait(i, polls);
        if (!arrived) s_fail = 1;
        __syncthreads();
        const bool ok = s_fail == 0;
        if (!ok) polls = 1;// a CTA that gave up keeps walking (its cluster waits for it at the barriers) without waiting again
        const uint4 *row = reinterpret_cast<const uint4 *>(rg.stage(i));
        float ss = 0.f;
        if (ok) {
            for (uint32_t v = threadIdx.x; v < nv; v += kThreads) {
                const uint4 q = row[v];
                const uint32_t *pw = reinterpret_cast<const uint32_t *>(&q);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = unpack2_t<DT>(pw[k]);
                    ss = fmaf(f.x, f.x, ss);
                    ss = fmaf(f.y, f.y, ss);
                }
            }
        }
        ss = cl > 1 ? cluster_reduce<false>(ss, red, &part, cl) : cta_reduce<false>(ss, red);
        if (ok) {
            const auto k = scale_of(ss, d, eps);
            uint16_t *yr = y + (int64_t) row_of(i) * stride_y + (size_t) v0 * 8;
            for (uint32_t v = threadIdx.x; v < nv; v += kThreads) {
                const uint4 q = row[v];
                st_stream(yr + (size_t) v * 8, prod(k, q, w, v0 + v));
            }
        }
        if (cl > 1) cluster_sync_all();// also: every thread of this CTA has read the stage
        else __syncthreads();
        if (threadIdx.x == 0 && ok && i + kStages < cnt) {
            rg.request(i + kStages, x + (int64_t) row_of(i + kStages) * stride_x + (size_t) v0 * 8, nv * 16u);
        }
    }
    if (threadIdx.x == 0 && s_fail) {
        // requests still in flight towards this CTA's shared memory: let them land (bounded) before it is given back
        for (uint32_t i = 0; i < cnt; ++i) {
            if (!mbar_wait_bounded(&full[i % kStages], (i / kStages) & 1u, 1u << 16)) break;
        }
        atomicAdd(&g_row_ring_timeouts, 1u);
    }
}

// ---------------------------------------------------------------- causal softmax --
// Rows are (batch, query row) pairs; row i of a batch entry sees `vis` columns, only those are requested.
template<int DT>
__device__ __forceinline__ void causal_softmax_ring_body(uint16_t *y, uint64_t rows, uint64_t seq_len, uint64_t total,
                                                         uint32_t vecs, int64_t stride_b, int64_t stride_i, Plan plan) {
    extern __shared__ __align__(128) unsigned char ring_smem[];
    __shared__ __align__(8) uint64_t full[kStages];
    __shared__ float red_m[32], red_s[32];
    __shared__ float part_m, part_s;
    __shared__ int s_fail;
    const uint32_t cl = plan.cl, rank = cl > 1 ? cluster_rank() : 0;
    const uint32_t clusters = gridDim.x / cl, me = blockIdx.x / cl;
    const uint32_t v0 = rank * plan.part_vecs;
    const uint32_t nv_all = v0 >= vecs ? 0u : (vecs - v0 < plan.part_vecs ? vecs - v0 : plan.part_vecs);
    const uint32_t cnt = me < rows ? (uint32_t) ((rows - me + clusters - 1) / clusters) : 0u;
    const Ring rg{full, ring_smem, plan.part_vecs * 16u};
    auto row_of = [&](uint32_t i) { return (uint64_t) me + (uint64_t) i * clusters; };
    auto row_ptr = [&](uint64_t row, uint32_t &vis) {
        const uint64_t b = row / seq_len, qi = row - b * seq_len;
        const uint64_t last = total - seq_len + qi;// wraps like the reference when seq_len > total
        vis = (uint32_t) (last >= total - 1 ? total : last + 1);
        return y + (int64_t) b * stride_b + (int64_t) qi * stride_i;
    };
    // vectors of this CTA's part that hold at least one visible column
    auto visible_vecs = [&](uint32_t vis) {
        const uint32_t upto = (vis + 7u) / 8u;
        return upto <= v0 ? 0u : (upto - v0 < nv_all ? upto - v0 : nv_all);
    };
    constexpr uint32_t kNegInf1 = DT == kBF16 ? 0xFF80u : 0xFC00u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (uint32_t i = 0; i < cnt && i < (uint32_t) kStages; ++i) {
            uint32_t vis;
            const uint16_t *p = row_ptr(row_of(i), vis);
            rg.request(i, p + (size_t) v0 * 8, visible_vecs(vis) * 16u);
        }
    }
    __syncthreads();
    uint32_t polls = kWaitPolls;
    for (uint32_t i = 0; i < cnt; ++i) {
        const bool arrived = rg.wait(i, polls);
        if (!arrived) s_fail = 1;
        __syncthreads();
        const bool ok = s_fail == 0;
        if (!ok) polls = 1;
        uint32_t vis;
        uint16_t *yr = row_ptr(row_of(i), vis) + (size_t) v0 * 8;
        const uint32_t nvis = visible_vecs(vis);
        const uint4 *row = reinterpret_cast<const uint4 *>(rg.stage(i));
        // element e of this CTA's part is column v0 * 8 + e; columns >= vis are masked
        auto load_masked = [&](uint32_t v, float *f) {
            const uint4 q = row[v];
            const uint32_t *pw = reinterpret_cast<const uint32_t *>(&q);
            const uint32_t col = (v0 + v) * 8u;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 t = unpack2_t<DT>(pw[k]);
                f[2 * k] = col + 2 * k < vis ? t.x : -INFINITY;
                f[2 * k + 1] = col + 2 * k + 1 < vis ? t.y : -INFINITY;
            }
        };
        (void) kNegInf1;
        float m = -INFINITY;
        if (ok) {
            for (uint32_t v = threadIdx.x; v < nvis; v += kThreads) {
                float f[8];
                load_masked(v, f);
#pragma unroll
                for (int k = 0; k < 8; ++k) m = fmaxf(m, f[k]);
            }
        }
        m = cl > 1 ? cluster_reduce<true>(m, red_m, &part_m, cl) : cta_reduce_alt<true>(m, red_m);
        const float mk = -m * kLog2e;
        float s = 0.f;
        if (ok) {
            for (uint32_t v = threadIdx.x; v < nvis; v += kThreads) {
                float f[8];
                load_masked(v, f);
#pragma unroll
                for (int k = 0; k < 8; ++k) s += fast_exp2(fmaf(f[k], kLog2e, mk));
            }
        }
        s = cl > 1 ? cluster_reduce<false>(s, red_s, &part_s, cl) : cta_reduce_alt<false>(s, red_s);
        if (ok) {
            const float r = __frcp_rn(s);
            for (uint32_t v = threadIdx.x; v < nv_all; v += kThreads) {
                uint4 out = make_uint4(0u, 0u, 0u, 0u);// masked columns: exact zeros
                if (v < nvis) {
                    float f[8];
                    load_masked(v, f);
                    uint32_t *po = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float q0 = __fmul_rn(fast_exp2(fmaf(f[2 * k], kLog2e, mk)), r);
                        const float q1 = __fmul_rn(fast_exp2(fmaf(f[2 * k + 1], kLog2e, mk)), r);
                        if (DT == kBF16) po[k] = (__float_as_uint(q0) >> 16) | (__float_as_uint(q1) & 0xFFFF0000u);
                        else asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(po[k]) : "f"(q1), "f"(q0));
                    }
                }
                st_stream(yr + (size_t) v * 8, out);
            }
        }
        if (cl > 1) cluster_sync_all();
        else __syncthreads();
        if (threadIdx.x == 0 && ok && i + kStages < cnt) {
            uint32_t vn;
            const uint16_t *p = row_ptr(row_of(i + kStages), vn);
            rg.request(i + kStages, p + (size_t) v0 * 8, visible_vecs(vn) * 16u);
        }
    }
    if (threadIdx.x == 0 && s_fail) {
        for (uint32_t i = 0; i < cnt; ++i) {
            if (!mbar_wait_bounded(&full[i % kStages], (i / kStages) & 1u, 1u << 16)) break;
        }
        atomicAdd(&g_row_ring_timeouts, 1u);
    }
}

}// namespace ring
}// namespace b200
