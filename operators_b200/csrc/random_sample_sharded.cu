// Vocabulary-sharded random sample: the two device stages on either side of the
// single all-gather.  No counterpart in the reference (it has no multi-device
// code at all); per-row semantics aim at the reference CPU backend's
// (src/ops/random_sample/cpu/random_sample.cc:45-129) applied to the
// concatenation of the shards.
//
//   stage 1 (every rank, its own columns [shard_offset, shard_offset + voc_local)):
//       per row -> one fixed-size record: local maximum, local sum of
//       exp((v - M_local)/T) and, in index order, every element >= a lower bound
//       of the local k-th largest value (those are a superset of the shard's
//       share of the global top-k, ties included).
//   all-gather of the records (~1 KB per row per rank), done by the host with
//       NCCL; records land in local memory before stage 2 reads them.
//   stage 2 (any rank): global maximum, rescaled sum, streaming insertion of the
//       gathered candidates in rank (= index) order with the reference's tie
//       rule, truncated probabilities, top-p cut, pick.
//
// What is exact and what is not: the top-k set, its tie order and the
// numerators are those of the CPU path.  The denominator is the correctly
// rounded sum; the CPU path's sequential fp32 sum is ~3e-4 smaller (it drops
// terms below half an ulp of the running sum), which moves a truncated fp16
// probability in about half of the rows and the sampled index in roughly one
// row per thousand.  Reproducing that sum needs the running value to travel
// from shard to shard and is not possible with one all-gather; the unsharded
// kernel does reproduce it.
#include "common.cuh"
#include "random_sample.cuh"
#include "random_sample_device.cuh"

#include "../../include/infiniop_ext.h"

using namespace b200;

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kListCap = 64;
constexpr int kRecCap = 128;               // candidates per record
constexpr int kRecHeader = 8;              // u32 words: count, max key, sum (2), reserved (4)
constexpr int kRecWords = kRecHeader + 2 * kRecCap;
constexpr uint32_t kOverflow = 0xFFFFFFFFu;


struct LocalShared {
    uint32_t list_idx[kWarps][kListCap];
    uint16_t list_key[kWarps][kListCap];
    int list_cnt[kWarps];
    int overflow;
    double red[kWarps];
};

__global__ void __launch_bounds__(kThreads, 1)
    sample_shard_local_kernel(const uint16_t *logits, int64_t row_stride, int n, uint32_t shard_offset, int topk,
                              float temperature, uint32_t *records) {
    __shared__ LocalShared sm;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint16_t *row = logits + (int64_t) blockIdx.x * row_stride;
    uint32_t *rec = records + (size_t) blockIdx.x * kRecWords;
    const bool aligned = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const uint32_t nvec = (uint32_t) (n + 7) / 8;

    auto load8 = [&](uint32_t vec, uint32_t keys[8]) {
        const uint32_t base = vec * 8;
        if (aligned && base + 8 <= (uint32_t) n) {
            const uint4 v = *reinterpret_cast<const uint4 *>(row + base);
            const uint32_t *p = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                keys[2 * q] = key_of((uint16_t) (p[q] & 0xFFFFu));
                keys[2 * q + 1] = key_of((uint16_t) (p[q] >> 16));
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) keys[e] = base + e < (uint32_t) n ? key_of(row[base + e]) : 0u;
        }
    };

    // pass 1: per-thread and row maximum
    uint32_t tmax = 0;
    for (uint32_t v = tid; v < nvec; v += kThreads) {
        uint32_t keys[8];
        load8(v, keys);
#pragma unroll
        for (int e = 0; e < 8; ++e) tmax = max(tmax, keys[e]);
    }
    if (tid < kWarps) sm.list_cnt[tid] = 0;
    if (tid == 0) sm.overflow = 0;
    int k = topk > n ? n : topk;
    uint32_t lo = 1, hi = 65535, mkey = 1;
    {
        const int have = __syncthreads_count(tmax >= 1);
        const int need = k < have ? k : have;
        while (lo < hi) {
            const uint32_t mid = (lo + hi + 1) >> 1;
            if (__syncthreads_count(tmax >= mid) >= need) lo = mid;
            else hi = mid - 1;
        }
        if (have < k) lo = 1;
        // row maximum: largest key any thread holds
        uint32_t a = 1, b = 65535;
        while (a < b) {
            const uint32_t mid = (a + b + 1) >> 1;
            if (__syncthreads_count(tmax >= mid) >= 1) a = mid;
            else b = mid - 1;
        }
        mkey = a;
    }
    const uint32_t L = lo;
    const float M = val_of(mkey);
    const float scale = kLog2e / temperature;
    const float mk = -M * scale;

    // pass 2: local sum of exp((v - M)/T) and ordered candidates, warp-contiguous spans
    double acc = 0.0;
    const uint32_t span = (nvec + kThreads - 1) / kThreads;// vectors per lane; a warp owns 32*span consecutive vectors
    for (uint32_t it = 0; it < span; ++it) {
        const uint32_t v = (warp * span + it) * 32 + lane;
        uint32_t keys[8];
        uint32_t mask = 0;
        float part = 0.f;
        if (v < nvec) {
            load8(v, keys);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (keys[e] != 0) part += fast_exp2(fmaf(val_of(keys[e]), scale, mk));
                mask |= (keys[e] >= L ? 1u : 0u) << e;
            }
        }
        acc += (double) part;
        // ordered append (index order inside the warp's span)
        const uint32_t any = __ballot_sync(0xffffffffu, mask != 0);
        if (any) {
            const int cnt = __popc(mask);
            int pre = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, pre, o);
                if (lane >= o) pre += t;
            }
            const int total = __shfl_sync(0xffffffffu, pre, 31);
            const int start = sm.list_cnt[warp];
            if (start + total > kListCap) {
                if (lane == 0) sm.overflow = 1;
            } else {
                int at = start + pre - cnt;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    if (mask & (1u << e)) {
                        sm.list_idx[warp][at] = shard_offset + v * 8 + e;
                        sm.list_key[warp][at] = (uint16_t) keys[e];
                        ++at;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) sm.list_cnt[warp] = min(start + total, kListCap + 1);
            __syncwarp();
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) sm.red[warp] = acc;
    __syncthreads();
    if (warp == 0) {
        // concatenate the warp lists in warp (= index) order
        int total = 0;
        bool over = sm.overflow != 0;
        for (int w = 0; w < kWarps && !over; ++w) {
            const int cnt = sm.list_cnt[w];
            if (total + cnt > kRecCap) {
                over = true;
                break;
            }
            for (int c = lane; c < cnt; c += 32) {
                rec[kRecHeader + 2 * (total + c)] = sm.list_idx[w][c];
                rec[kRecHeader + 2 * (total + c) + 1] = sm.list_key[w][c];
            }
            total += cnt;
        }
        if (lane == 0) {
            double s = 0.0;
            for (int w = 0; w < kWarps; ++w) s += sm.red[w];
            rec[0] = over ? kOverflow : (uint32_t) total;
            rec[1] = mkey;
            rec[2] = (uint32_t) (__double_as_longlong(s) & 0xFFFFFFFFll);
            rec[3] = (uint32_t) ((unsigned long long) __double_as_longlong(s) >> 32);
            rec[4] = rec[5] = rec[6] = rec[7] = 0;
        }
    }
}

// One warp per row.  records: [ranks][rows][kRecWords].
__global__ void __launch_bounds__(128)
    sample_shard_finish_kernel(const uint32_t *records, int ranks, int rows, const float *random_vals, float topp,
                               int topk, float temperature, int voc_total, uint64_t *results, int *status) {
    __shared__ uint32_t s_key[4][kSlots];
    __shared__ uint32_t s_idx[4][kSlots];
    __shared__ float s_p[4][kSlots];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int row = blockIdx.x * 4 + w;
    if (row >= rows) return;
    const int k = topk > voc_total ? voc_total : topk;

    uint32_t mkey = 1;
    bool bad = false;
    for (int r = 0; r < ranks; ++r) {
        const uint32_t *rec = records + ((size_t) r * rows + row) * kRecWords;
        mkey = max(mkey, rec[1]);
        bad |= rec[0] == kOverflow;
    }
    if (bad) {
        if (lane == 0) atomicExch(status, 1);
        return;
    }
    const float M = val_of(mkey);
    double S = 0.0;
    TopBuf tb{0, 0, 0, 0};
    for (int r = 0; r < ranks; ++r) {
        const uint32_t *rec = records + ((size_t) r * rows + row) * kRecWords;
        const double sr = __longlong_as_double((long long) (((unsigned long long) rec[3] << 32) | rec[2]));
        const float dx = __fdiv_rn(__fsub_rn(val_of(rec[1]), M), temperature);
        S += sr * exp((double) dx);
        const int cnt = (int) rec[0];
        for (int c = 0; c < cnt; ++c) {
            topbuf_insert(tb, lane, k, rec[kRecHeader + 2 * c + 1], rec[kRecHeader + 2 * c]);
        }
    }
    s_key[w][lane] = tb.k0;
    s_key[w][lane + 32] = tb.k1;
    s_idx[w][lane] = tb.i0;
    s_idx[w][lane + 32] = tb.i1;
    __syncwarp();
    const float Sf = (float) S;
    for (int i = lane; i < k; i += 32) {
        const float t = term_of(val_of(s_key[w][i]), M, temperature);
        s_p[w][i] = f16_to_f32(f32_to_f16_ref(__fdiv_rn(t, Sf)));
    }
    __syncwarp();
    if (lane == 0) pick_from_topk(s_p[w], s_idx[w], k, topp, random_vals[row], results + row);
}

}// namespace

INFINIOP_API uint64_t infiniopRandomSampleShardRecordBytes(void) { return (uint64_t) kRecWords * 4; }

INFINIOP_API infiniopStatus_t infiniopRandomSampleShardLocal(infiniopRandomSampleDescriptor_t desc, void *records,
                                                             void const *logits, int64_t row_stride, uint64_t rows,
                                                             uint64_t shard_offset, int topk, float temperature,
                                                             void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (records == nullptr || logits == nullptr) return STATUS_BAD_PARAM;
    if (rows == 0) return STATUS_SUCCESS;
    auto *d = reinterpret_cast<RandomSampleDesc *>(desc);
    if (rows > 0x7FFFFFFFull || shard_offset > 0xFFFFFFFFull - (uint64_t) d->voc) return STATUS_BAD_PARAM;
    if (topk < 1 || topk > kSlots || !(temperature > 0.f)) return STATUS_BAD_PARAM;
    DeviceGuard guard(d->device_id);
    sample_shard_local_kernel<<<(uint32_t) rows, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint16_t *>(logits), row_stride, d->voc, (uint32_t) shard_offset, topk, temperature,
        reinterpret_cast<uint32_t *>(records));
    return check_launch("random_sample_shard_local");
}

INFINIOP_API infiniopStatus_t infiniopRandomSampleShardFinish(infiniopHandle_t handle, void *results,
                                                              void const *gathered_records, int ranks, uint64_t rows,
                                                              uint64_t voc_total, void const *random_vals, float topp,
                                                              int topk, float temperature, void *status_flag,
                                                              void *stream) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (results == nullptr || gathered_records == nullptr || random_vals == nullptr || status_flag == nullptr) {
        return STATUS_BAD_PARAM;
    }
    if (rows == 0) return STATUS_SUCCESS;
    if (ranks < 1 || rows > 0x7FFFFFFFull || voc_total == 0 || voc_total > 0x7FFFFFFFull) return STATUS_BAD_PARAM;
    if (topk < 2 || topk > kSlots || !(topp > 0.f) || !(temperature > 0.f)) return STATUS_BAD_PARAM;
    auto *h = reinterpret_cast<Handle *>(handle);
    DeviceGuard guard(h->device_id);
    const uint32_t grid = (uint32_t) ((rows + 3) / 4);
    sample_shard_finish_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint32_t *>(gathered_records), ranks, (int) rows,
        reinterpret_cast<const float *>(random_vals), topp, topk, temperature, (int) voc_total,
        reinterpret_cast<uint64_t *>(results), reinterpret_cast<int *>(status_flag));
    return check_launch("random_sample_shard_finish");
}
