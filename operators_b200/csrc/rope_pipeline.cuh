// RoPE for contiguous token rows: persistent CTAs, one per SM, in which every
// group of warps streams its own tokens through its own ring of shared-memory stages with
// bulk asynchronous copies (TMA, cp.async.bulk) that complete on mbarriers.
//
// Why: with one short-lived CTA per token pair all CTAs of a wave load, then
// compute, then store in step, and the pos -> table row -> arithmetic chain sits
// in front of every store; the memory system idles during the arithmetic.  Here
// each group of warps keeps kStagesPerGroup token rows (and their sin/cos rows)
// in flight, rotates whatever has landed and sends it back with a bulk store that
// drains while the next rows are worked on.  Groups never wait for one another:
// there is no CTA barrier in the loop, only the group's own named barrier.
//
// Per token the stage holds [row: nhead*dh fp16][sin row: dh fp32][cos row: dh
// fp32].  All three copies signal the stage's mbarrier through their byte
// counts.  A stage is refilled only after the bulk store that read it has
// finished reading (cp.async.bulk.wait_group.read; bulk groups are per thread,
// and one thread of the group issues all of its copies).
//
// Every wait on an mbarrier is bounded: when a copy does not arrive within the
// limit (g_rope_wait_polls tries) the group stops rotating, waits for the copies
// it still has in flight (with the full default limit), drains its stores,
// counts itself in g_rope_pipeline_timeouts and leaves; nothing spins forever.
// A non-zero counter means rows were left un-rotated although the call returned
// STATUS_SUCCESS; the host reads it through infiniopExtDeviceTimeouts.
#pragma once

#include "bulk_copy.cuh"
#include "common.cuh"

namespace b200 {
namespace rope_pipe {

using namespace bulk;

// measured at [4096, 32, 128] (kernel duration, cold L2): 32 warps in groups of 4 -> 16.4 us, 24 in groups of 3 -> 17.2,
// 16 in groups of 2 -> 19.0, 32 in groups of 8 -> 19.3; the same pipeline without the arithmetic 13.1; with the
// packed fp32 instructions (mul / add .f32x2) the instruction count stays the same and the kernel takes 18.7
constexpr int kWarpsPerCta = 32;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kWarpsPerGroup = 4;         // warps that share one ring of stages and split each token row
constexpr int kGroups = kWarpsPerCta / kWarpsPerGroup;
constexpr int kTotalStages = 24;          // 24 x 9 KB for rows of 32 heads x 128 (16 stages: 17.7 us, 24: 16.5 us)
constexpr int kStagesPerGroup = kTotalStages / kGroups;
constexpr int kGroupThreads = kWarpsPerGroup * 32;
static_assert(kStagesPerGroup >= 2 && kGroups <= 15, "a ring needs two stages; named barriers 1..15");
constexpr int kMaxTokensPerGroup = 32;    // a lane of the group's first warp keeps the position id of one of its tokens

__device__ unsigned int g_rope_pipeline_timeouts = 0;
__device__ unsigned int g_rope_wait_polls = kWaitPolls;// settable from the host (infiniopExtSetWaitLimit)

// Stage layout and the launch geometry, worked out once on the host.
struct Plan {
    uint32_t row_bytes;  // nhead * dh * 2
    uint32_t tab_bytes;  // dh * 4
    uint32_t stage_bytes;// row + 2 tables, a multiple of 128
    uint32_t slices;     // 16-byte vectors per head: divides 32, so a lane stays on one slice
    uint32_t row_vecs;   // 16-byte vectors per token row
    uint32_t grid;
    size_t smem_bytes;   // kTotalStages stages
};

__device__ __forceinline__ void group_barrier(int group) {
    if (kWarpsPerGroup == 1) __syncwarp();
    else asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kGroupThreads) : "memory");
}

// t rows contiguous ([tokens] x nhead*dh halves, token stride >= row, all 16-byte aligned).
// Token order: group g of CTA c takes tokens c + G * (g + kGroups * j), j = 0, 1, ...
// DIRECT: the rotated vectors are stored to global memory by the threads themselves; otherwise they go back into the
// stage and one bulk copy returns the row.
template<int DT, bool DIRECT>
__global__ void __launch_bounds__(kThreads, 1)
rope_pipeline_kernel(uint16_t *t, const uint64_t *pos_ids, const float *sin_table, const float *cos_table, uint32_t seq_len,
                     uint32_t dim, int64_t stride_0, Plan plan) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full_bar[kGroups][kStagesPerGroup];
    __shared__ int s_fail[kGroups];

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, G = gridDim.x, c = blockIdx.x;
    const uint32_t group = warp / kWarpsPerGroup, gtid = threadIdx.x - group * kGroupThreads;// thread within the group
    const bool issuer = gtid == 0;                                                           // issues all of the group's copies
    auto token_of = [&](uint32_t j) { return (uint64_t) c + (uint64_t) G * (group + (uint64_t) kGroups * j); };
    uint32_t cnt = 0;// this group's tokens
    {
        const uint64_t first_tok = token_of(0), step = (uint64_t) G * kGroups;
        if (first_tok < seq_len) cnt = (uint32_t) ((seq_len - first_tok + step - 1) / step);
    }
    unsigned char *my_smem = smem + (size_t) group * kStagesPerGroup * plan.stage_bytes;
    auto stage_ptr = [&](uint32_t s) { return my_smem + (size_t) s * plan.stage_bytes; };
    auto row_of = [&](uint32_t j) { return t + (int64_t) token_of(j) * stride_0; };
    uint64_t *bar = full_bar[group];

    if (issuer) {
        for (int s = 0; s < kStagesPerGroup; ++s) mbar_init(&bar[s], 1);
        s_fail[group] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    group_barrier(group);
    // The rows of the first tokens do not depend on the position ids: start them now.
    const uint32_t first = cnt < (uint32_t) kStagesPerGroup ? cnt : (uint32_t) kStagesPerGroup;
    if (issuer) {
        for (uint32_t j = 0; j < first; ++j) {
            mbar_expect_tx(&bar[j], plan.row_bytes + 2 * plan.tab_bytes);
            bulk_load(stage_ptr(j), row_of(j), plan.row_bytes, &bar[j]);
        }
    }
    // lane j of the group's first warp holds the position of the group's token j
    const uint64_t my_pos = (gtid < 32 && lane < cnt) ? pos_ids[token_of(lane)] : 0;
    auto load_tables = [&](uint64_t p, uint32_t s) {// issuer
        bulk_load(stage_ptr(s) + plan.row_bytes, sin_table + p * dim, plan.tab_bytes, &bar[s]);
        bulk_load(stage_ptr(s) + plan.row_bytes + plan.tab_bytes, cos_table + p * dim, plan.tab_bytes, &bar[s]);
    };
    for (uint32_t j = 0; j < first; ++j) {
        const uint64_t p = __shfl_sync(0xffffffffu, my_pos, j);
        if (issuer) load_tables(p, j);
    }

    const uint32_t slice = lane % plan.slices;// this lane's 8 positions of the head dimension
    const uint32_t polls = *reinterpret_cast<volatile unsigned int *>(&g_rope_wait_polls);
    bool failed = false;
    uint32_t j_fail = 0;
    for (uint32_t j = 0; j < cnt; ++j) {
        const uint32_t s = j % kStagesPerGroup, parity = (j / kStagesPerGroup) & 1u;
        const bool arrived = mbar_wait_bounded(&bar[s], parity, polls);
        if (!__all_sync(0xffffffffu, arrived)) s_fail[group] = 1;// seen by the whole group after its barrier
        unsigned char *st = stage_ptr(s);
        if (arrived) {
            const float4 *sn4 = reinterpret_cast<const float4 *>(st + plan.row_bytes) + slice * 2;
            const float4 *cs4 = reinterpret_cast<const float4 *>(st + plan.row_bytes + plan.tab_bytes) + slice * 2;
            const float4 s0 = sn4[0], s1 = sn4[1], c0 = cs4[0], c1 = cs4[1];
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            uint4 *row = reinterpret_cast<uint4 *>(st);
            uint16_t *grow = row_of(j);
#pragma unroll 8
            for (uint32_t v = gtid; v < plan.row_vecs; v += kGroupThreads) {
                const uint4 q = row[v];
                uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 ab = unpack2_t<DT>(w[k]);
                    const float r0 = __fsub_rn(__fmul_rn(ab.x, cs[2 * k]), __fmul_rn(ab.y, sn[2 * k]));
                    const float r1 = __fadd_rn(__fmul_rn(ab.x, sn[2 * k + 1]), __fmul_rn(ab.y, cs[2 * k + 1]));
                    w[k] = pack2_t<DT>(r0, r1);
                }
                if (DIRECT) st_stream(grow + (size_t) v * 8, make_uint4(w[0], w[1], w[2], w[3]));
                else row[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        if (!DIRECT) fence_async_shared();
        group_barrier(group);// every thread of the group has read (and, with bulk stores, rewritten) stage s
        if (s_fail[group]) {// the same decision in every thread of the group
            failed = true;
            j_fail = j;
            break;
        }
        if (DIRECT) {
            // Stage s is free again: it takes token j + kStagesPerGroup.
            const uint32_t jn = j + kStagesPerGroup;
            const bool refill = jn < cnt;
            const uint64_t pn = __shfl_sync(0xffffffffu, my_pos, jn & 31u);
            if (issuer && refill) {
                mbar_expect_tx(&bar[s], plan.row_bytes + 2 * plan.tab_bytes);
                bulk_load(stage_ptr(s), row_of(jn), plan.row_bytes, &bar[s]);
                load_tables(pn, s);
            }
        } else {
            // The stage used by token j - 1 is free once its store has read it; it takes token j - 1 + kStagesPerGroup.
            const uint32_t jn = j + kStagesPerGroup - 1;
            const bool refill = j >= 1 && jn < cnt;
            const uint64_t pn = __shfl_sync(0xffffffffu, my_pos, jn & 31u);
            if (issuer) {
                bulk_store(row_of(j), st, plan.row_bytes);
                bulk_commit();
                if (refill) {
                    bulk_wait_read<1>();
                    const uint32_t sr = (j - 1) % kStagesPerGroup;
                    mbar_expect_tx(&bar[sr], plan.row_bytes + 2 * plan.tab_bytes);
                    bulk_load(stage_ptr(sr), row_of(jn), plan.row_bytes, &bar[sr]);
                    load_tables(pn, sr);
                }
            }
        }
    }
    if (issuer) {
        if (failed) {
            // the loads of tokens j_fail .. are still in flight towards this CTA's shared memory: let them land
            // before the CTA gives the memory back (token i + kStagesPerGroup is requested at the end of pass i)
            uint32_t issued = DIRECT ? j_fail + kStagesPerGroup : (j_fail == 0 ? first : j_fail + kStagesPerGroup - 1);
            if (issued > cnt) issued = cnt;
            for (uint32_t jj = j_fail; jj < issued; ++jj) {
                mbar_wait_bounded(&bar[jj % kStagesPerGroup], (jj / kStagesPerGroup) & 1u);
            }
            atomicAdd(&g_rope_pipeline_timeouts, 1u);
        }
        if (!DIRECT) bulk_wait_all();
    }
}

}// namespace rope_pipe
}// namespace b200
