// Rotary position embedding, in place on t[tokens, heads, dh] fp16.
//
// Replaces reference src/ops/rotary_embedding/cuda/rotary_embedding.cu:5-68 and
// src/ops/rotary_embedding/cuda/rotary_embedding.cc:5-65 behind
// include/ops/rotary_embedding/rotary_embedding.h.  Arithmetic follows the CPU
// backend (src/ops/rotary_embedding/cpu/rotary_embedding_cpu.cc:16-44): for the
// pair (a, b) = (t[2k], t[2k+1]) of token i with p = pos_ids[i],
//   t[2k]   = trunc16(a * cos[p*dh + 2k]     - b * sin[p*dh + 2k])
//   t[2k+1] = trunc16(a * sin[p*dh + 2k + 1] + b * cos[p*dh + 2k + 1])
// with un-fused fp32 multiplies and adds, so results are bit-identical.  As in
// the reference the table row offset is p * dh (the table's own row stride is
// not used) and p is not range-checked.
//
// t is read and written once; a token's two table rows are read from HBM once
// and shared by all its heads.  Two kernels:
//  * rope_pipeline_kernel (rope_pipeline.cuh): contiguous token rows go through
//    shared memory with bulk asynchronous copies, persistent CTAs, no CTA
//    barrier in the loop.  Taken whenever the layout allows it.
//  * rope_kernel (below): any strides.  Thread -> (token, slice of the head
//    dimension); the thread keeps its slice of the sin/cos rows in registers
//    and walks over the heads with several 128-bit loads in flight.  The
//    environment variable INFINIOP_ROPE_KERNEL (any value) forces this one.
//
// rope_kernel also serves infiniopRoPERearrange (not in the reference): the
// rotated values of `src` are written to a second view `dst` of the same shape
// with its own strides, e.g. the rows of the K cache at the tokens' positions,
// so the rotation and the cache write (reference src/ops/attention/operator.cc:
// 87-91: a rearrange of k into k_cache) cost one pass over k instead of two.
#include "common.cuh"
#include "rope_pipeline.cuh"

#include <cstdlib>
#include <new>

using namespace b200;

namespace {

struct RoPEDesc {
    Device device;
    int device_id;
    int sm_count;
    int max_smem_optin;
    uint64_t seq_len, nhead, dim;
    int64_t stride_0, stride_1;
    bool to_dst;                 // RoPERearrange: rotated values go to a second view
    int64_t dstride_0, dstride_1;
    int dt;                      // kF16, or kBF16 (an extension: bf16 storage, the same un-fused fp32 arithmetic)
};

// One slice = V halves of one head (V = 8: a 128-bit vector, V = 2: one pair).
// ALIGNED says whether a slice may be moved with a single V*2-byte access.
template<int V, bool ALIGNED>
struct Slice {
    uint32_t w[V / 2];// V / 2 packed pairs
    __device__ __forceinline__ void load(const uint16_t *p) {
        if (ALIGNED && V == 8) {
            const uint4 q = ld_stream(p);
            w[0] = q.x, w[V / 2 > 1 ? 1 : 0] = q.y, w[V / 2 > 2 ? 2 : 0] = q.z, w[V / 2 > 3 ? 3 : 0] = q.w;
        } else if (ALIGNED) {
#pragma unroll
            for (int e = 0; e < V / 2; ++e) w[e] = reinterpret_cast<const uint32_t *>(p)[e];
        } else {
#pragma unroll
            for (int e = 0; e < V / 2; ++e) w[e] = (uint32_t) p[2 * e] | ((uint32_t) p[2 * e + 1] << 16);
        }
    }
    __device__ __forceinline__ void store(uint16_t *p) const {
        if (ALIGNED && V == 8) {
            st_stream(p, make_uint4(w[0], w[V / 2 > 1 ? 1 : 0], w[V / 2 > 2 ? 2 : 0], w[V / 2 > 3 ? 3 : 0]));
        } else if (ALIGNED) {
#pragma unroll
            for (int e = 0; e < V / 2; ++e) reinterpret_cast<uint32_t *>(p)[e] = w[e];
        } else {
#pragma unroll
            for (int e = 0; e < V / 2; ++e) {
                p[2 * e] = (uint16_t) w[e];
                p[2 * e + 1] = (uint16_t) (w[e] >> 16);
            }
        }
    }
};

constexpr int kHeadsInFlight = 4;// measured at [4096,32,128]: 4 -> 23 us, 2 -> 27 us, 8 -> 29 us

// Block = tokens_per_cta x threads_per_token.  threads_per_token is a multiple
// of slices_per_head, so a thread's slice index within the head never changes
// while it strides over (head, slice) items: its table values load once.
template<int V, bool ALIGNED, int DT>
__global__ void __launch_bounds__(256, 4) rope_kernel(uint16_t *dst, const uint16_t *t, const uint64_t *pos_ids, const float *sin_table, const float *cos_table,
                            uint64_t seq_len, uint32_t nhead, uint32_t dim, int64_t stride_0, int64_t stride_1,
                            int64_t dstride_0, int64_t dstride_1, uint32_t threads_per_token, uint32_t slices_per_head) {
    const uint32_t tok_in_cta = threadIdx.x / threads_per_token;
    const uint32_t lt = threadIdx.x - tok_in_cta * threads_per_token;
    const uint32_t tokens_per_cta = blockDim.x / threads_per_token;
    // Usual case: the token's threads cover every slice of a head at least once
    // and a thread keeps one slice.  Very wide heads (more slices than threads):
    // a thread walks over slices as well and visits every head.
    const bool wide = threads_per_token < slices_per_head;
    const uint32_t slice0 = wide ? lt : lt % slices_per_head;
    const uint32_t slice_step = wide ? threads_per_token : slices_per_head;
    const uint32_t head0 = wide ? 0 : lt / slices_per_head;
    const uint32_t head_step = wide ? 1 : threads_per_token / slices_per_head;

    for (uint64_t tok = (uint64_t) blockIdx.x * tokens_per_cta + tok_in_cta; tok < seq_len;
         tok += (uint64_t) gridDim.x * tokens_per_cta) {
        const uint64_t p = pos_ids[tok];
        for (uint32_t slice = slice0; slice < slices_per_head; slice += slice_step) {
            const uint16_t *base = t + (int64_t) tok * stride_0 + slice * V;
            uint16_t *out = dst + (int64_t) tok * dstride_0 + slice * V;
            // First group of heads goes in flight before the position id is
            // needed: the pos -> table-address -> table-load chain then overlaps
            // with the loads of t instead of preceding them.
            Slice<V, ALIGNED> x[kHeadsInFlight];
#pragma unroll
            for (int u = 0; u < kHeadsInFlight; ++u) {
                const uint32_t hh = head0 + u * head_step;
                if (hh < nhead) x[u].load(base + (int64_t) hh * stride_1);
            }
            const float *sr = sin_table + p * dim + slice * V;
            const float *cr = cos_table + p * dim + slice * V;
            float sn[V], cs[V];
            if constexpr (V == 8) {
                const float4 s0 = __ldg(reinterpret_cast<const float4 *>(sr)), s1 = __ldg(reinterpret_cast<const float4 *>(sr) + 1);
                const float4 c0 = __ldg(reinterpret_cast<const float4 *>(cr)), c1 = __ldg(reinterpret_cast<const float4 *>(cr) + 1);
                sn[0] = s0.x, sn[1] = s0.y, sn[2] = s0.z, sn[3] = s0.w, sn[4] = s1.x, sn[5] = s1.y, sn[6] = s1.z, sn[7] = s1.w;
                cs[0] = c0.x, cs[1] = c0.y, cs[2] = c0.z, cs[3] = c0.w, cs[4] = c1.x, cs[5] = c1.y, cs[6] = c1.z, cs[7] = c1.w;
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    sn[e] = __ldg(sr + e);
                    cs[e] = __ldg(cr + e);
                }
            }
            for (uint32_t h = head0; h < nhead; h += head_step * kHeadsInFlight) {
#pragma unroll
                for (int u = 0; u < kHeadsInFlight; ++u) {
                    const uint32_t hh = h + u * head_step;
                    if (hh < nhead) {
#pragma unroll
                        for (int k = 0; k < V / 2; ++k) {
                            const float2 ab = unpack2_t<DT>(x[u].w[k]);
                            const float r0 = __fsub_rn(__fmul_rn(ab.x, cs[2 * k]), __fmul_rn(ab.y, sn[2 * k]));
                            const float r1 = __fadd_rn(__fmul_rn(ab.x, sn[2 * k + 1]), __fmul_rn(ab.y, cs[2 * k + 1]));
                            x[u].w[k] = pack2_t<DT>(r0, r1);// both halves with one truncating conversion
                        }
                        x[u].store(out + (int64_t) hh * dstride_1);
                    }
                }
                // next group of heads for this thread, if any
                const uint32_t hn = h + head_step * kHeadsInFlight;
#pragma unroll
                for (int u = 0; u < kHeadsInFlight; ++u) {
                    const uint32_t hh = hn + u * head_step;
                    if (hh < nhead) x[u].load(base + (int64_t) hh * stride_1);
                }
            }
        }
    }
}

}// namespace

namespace b200 {
// Groups of the bulk-copy pipeline that gave up on a wait since the library was loaded (synchronises the device).
unsigned long long rope_pipeline_timeouts_read() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, rope_pipe::g_rope_pipeline_timeouts, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return ~0ull;
    }
    return v;
}
// Tries per mbarrier wait of the pipeline; 0 restores the default.
bool rope_pipeline_set_wait_polls(unsigned int polls) {
    if (polls == 0) polls = rope_pipe::kWaitPolls;
    if (cudaMemcpyToSymbol(rope_pipe::g_rope_wait_polls, &polls, sizeof(polls)) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return true;
}
}// namespace b200

INFINIOP_API infiniopStatus_t infiniopCreateRoPEDescriptor(infiniopHandle_t handle, infiniopRoPEDescriptor_t *desc_ptr,
                                                           infiniopTensorDescriptor_t t,
                                                           infiniopTensorDescriptor_t pos_ids,
                                                           infiniopTensorDescriptor_t sin_table,
                                                           infiniopTensorDescriptor_t cos_table) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    // Checks, order and codes of reference rotary_embedding.cc:11-50.  The
    // reference's nv-gpu limit dh/2 <= 1024 (rotary_embedding.cc:35-37) comes from
    // its one-thread-per-pair launch and does not apply here.
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (t == nullptr || pos_ids == nullptr || sin_table == nullptr || cos_table == nullptr) return STATUS_BAD_PARAM;
    if (t->ndim != 3 || pos_ids->ndim != 1 || sin_table->ndim != 2 || cos_table->ndim != 2) return STATUS_BAD_TENSOR_SHAPE;
    const uint64_t seq_len = t->shape[0], nhead = t->shape[1], dim = t->shape[2];
    if (dim % 2 != 0) return STATUS_BAD_TENSOR_SHAPE;
    if (pos_ids->shape[0] != seq_len || sin_table->shape[1] != dim || cos_table->shape[1] != dim ||
        sin_table->shape[0] != cos_table->shape[0]) {
        return STATUS_BAD_TENSOR_SHAPE;
    }
    if (nhead > 0xFFFFFFFFull || dim > 0xFFFFFFFFull) return STATUS_BAD_TENSOR_SHAPE;
    if (t->strides[2] != 1 || pos_ids->strides[0] != 1 || sin_table->strides[1] != 1 || cos_table->strides[1] != 1) {
        return STATUS_BAD_TENSOR_STRIDES;
    }
    if (!dt_eq(t->dt, F16) && !dt_eq(t->dt, BF16)) return STATUS_BAD_TENSOR_DTYPE;// bf16: an extension
    if (!dt_eq(sin_table->dt, F32) || !dt_eq(cos_table->dt, F32)) return STATUS_BAD_TENSOR_DTYPE;
    if (!dt_eq(pos_ids->dt, U64)) return STATUS_BAD_TENSOR_DTYPE;

    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow)
        RoPEDesc{DevNvGpu, h->device_id, h->sm_count, h->max_smem_optin, seq_len, nhead, dim, t->strides[0], t->strides[1],
                 false,    0,            0,         store_type_of(t->dt)};
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    *desc_ptr = reinterpret_cast<infiniopRoPEDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetRoPEWorkspaceSize(infiniopRoPEDescriptor_t desc, uint64_t *size) {
    if (desc == nullptr) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = 0;
    return STATUS_SUCCESS;
}

namespace {

// Kernel choice and launch; `out` is `t` itself for the in-place operator.
infiniopStatus_t run(const RoPEDesc *d, void *out, const void *t, void const *pos_ids, void const *sin_table,
                     void const *cos_table, cudaStream_t st) {
    const bool in_place = !d->to_dst;
    const int64_t dstride_0 = in_place ? d->stride_0 : d->dstride_0, dstride_1 = in_place ? d->stride_1 : d->dstride_1;
    auto *tp = reinterpret_cast<uint16_t *>(const_cast<void *>(t));
    auto *op = reinterpret_cast<uint16_t *>(out);
    auto *pp = reinterpret_cast<const uint64_t *>(pos_ids);
    auto *sp = reinterpret_cast<const float *>(sin_table);
    auto *cp = reinterpret_cast<const float *>(cos_table);
    const uint32_t nhead = (uint32_t) d->nhead, dim = (uint32_t) d->dim;

    // Widest slice the layout allows: 8 halves need 16-byte aligned rows of t
    // and of both tables (dh % 8 == 0 makes p*dh*4 a multiple of 32 bytes).
    const bool v8 = dim % 8 == 0 && d->stride_0 % 8 == 0 && d->stride_1 % 8 == 0 && aligned16(t) &&
                    dstride_0 % 8 == 0 && dstride_1 % 8 == 0 && aligned16(out) && aligned16(sin_table) &&
                    aligned16(cos_table);
    // Contiguous token rows of a size that leaves room for a few stages: the bulk-copy pipeline.
    if (in_place && v8 && d->stride_1 == (int64_t) dim && d->seq_len <= 0xFFFFFFFFull &&
        kernel_choice(kFamilyRoPE) != 1) {
        namespace rp = rope_pipe;
        rp::Plan plan;
        plan.row_bytes = nhead * dim * 2u;
        plan.tab_bytes = dim * 4u;
        // Rotated vectors are stored by the threads themselves (measured back to back at [4096, 32, 128] / [16384, 32,
        // 128]: 16.4 / 52.6 us against 17.2 / 55.6 us when they go back into the stage and a bulk copy returns the row;
        // infiniopExtSelectKernel(rope, 2) keeps that form).  Padding the table rows in the stage against the two-way
        // bank conflicts of their reads costs more bulk copies than it saves: 17.1 / 54.0 us; left out.
        const bool direct = kernel_choice(kFamilyRoPE) != 2;
        plan.stage_bytes = (plan.row_bytes + 2u * plan.tab_bytes + 127u) & ~127u;
        plan.slices = dim / 8u;
        plan.row_vecs = plan.row_bytes / 16u;
        const uint64_t overflow_guard = (uint64_t) nhead * dim * 2ull;
        const uint32_t grid = (uint32_t) (d->seq_len < (uint64_t) d->sm_count ? d->seq_len : (uint64_t) d->sm_count);
        plan.grid = grid;
        plan.smem_bytes = (size_t) rp::kTotalStages * plan.stage_bytes;
        const uint64_t per_group = (d->seq_len + (uint64_t) grid * rp::kGroups - 1) / ((uint64_t) grid * rp::kGroups);
        // rows shorter than 4 KB (e.g. 8 heads of 128) leave the stages too small to pay: measured 10.3 us against
        // 7.0 us for the strided kernel at [4096, 8, 128]
        if (overflow_guard == plan.row_bytes && plan.row_bytes >= 4096u && plan.smem_bytes + 1024 <= (size_t) d->max_smem_optin &&
            32u % plan.slices == 0 &&
            per_group <= (uint64_t) rp::kMaxTokensPerGroup) {
            static thread_local int configured_dev = -1, configured_bytes = 0;
            if (configured_dev != d->device_id || configured_bytes < (int) plan.smem_bytes) {
                if (cudaFuncSetAttribute(rp::rope_pipeline_kernel<kF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int) plan.smem_bytes) != cudaSuccess ||
                    cudaFuncSetAttribute(rp::rope_pipeline_kernel<kF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int) plan.smem_bytes) != cudaSuccess ||
                    cudaFuncSetAttribute(rp::rope_pipeline_kernel<kBF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int) plan.smem_bytes) != cudaSuccess ||
                    cudaFuncSetAttribute(rp::rope_pipeline_kernel<kBF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int) plan.smem_bytes) != cudaSuccess) {
                    cudaGetLastError();
                    return STATUS_EXECUTION_FAILED;
                }
                configured_dev = d->device_id;
                configured_bytes = (int) plan.smem_bytes;
            }
            auto *kernel = d->dt == kBF16 ? (direct ? rp::rope_pipeline_kernel<kBF16, true> : rp::rope_pipeline_kernel<kBF16, false>)
                                          : (direct ? rp::rope_pipeline_kernel<kF16, true> : rp::rope_pipeline_kernel<kF16, false>);
            kernel<<<grid, rp::kThreads, plan.smem_bytes, st>>>(tp, pp, sp, cp, (uint32_t) d->seq_len, dim, d->stride_0, plan);
            return check_launch("rope_pipeline");
        }
    }
    const bool v2_aligned = d->stride_0 % 2 == 0 && d->stride_1 % 2 == 0 && aligned4(t) && dstride_0 % 2 == 0 &&
                            dstride_1 % 2 == 0 && aligned4(out);
    const uint32_t V = v8 ? 8 : 2;
    const uint32_t slices = dim / V;
    // threads per token: a multiple of `slices`, about (items / kHeadsInFlight)
    // so that every thread has a full set of loads in flight, capped at 256 (the kernel's launch bound).
    uint32_t heads_per_pass = (nhead + kHeadsInFlight - 1) / kHeadsInFlight;
    uint32_t tpt = slices * heads_per_pass;
    while (tpt > 256 && heads_per_pass > 1) {
        heads_per_pass = (heads_per_pass + 1) / 2;
        tpt = slices * heads_per_pass;
    }
    if (tpt > 256) tpt = 256;// more slices per head than a CTA has threads
    uint32_t tokens_per_cta = 1, threads = tpt;
    if (tpt < 256) {
        tokens_per_cta = 256 / tpt;
        threads = tokens_per_cta * tpt;
    }
    const uint64_t ctas = (d->seq_len + tokens_per_cta - 1) / tokens_per_cta;
    const uint64_t cap = 0x7FFFFFFFull;// one CTA per token group; more tokens than that loop
    const uint32_t grid = (uint32_t) (ctas < cap ? ctas : cap);
#define B200_ROPE_LAUNCH(V_, AL_, DT_)                                                                                    \
    rope_kernel<V_, AL_, DT_><<<grid, threads, 0, st>>>(op, tp, pp, sp, cp, d->seq_len, nhead, dim, d->stride_0, d->stride_1, \
                                                       dstride_0, dstride_1, tpt, slices)
    if (d->dt == kBF16) {
        if (v8) B200_ROPE_LAUNCH(8, true, kBF16);
        else if (v2_aligned) B200_ROPE_LAUNCH(2, true, kBF16);
        else B200_ROPE_LAUNCH(2, false, kBF16);
    } else {
        if (v8) B200_ROPE_LAUNCH(8, true, kF16);
        else if (v2_aligned) B200_ROPE_LAUNCH(2, true, kF16);
        else B200_ROPE_LAUNCH(2, false, kF16);
    }
#undef B200_ROPE_LAUNCH
    return check_launch("rope");
}

}// namespace

INFINIOP_API infiniopStatus_t infiniopRoPE(infiniopRoPEDescriptor_t desc, void *workspace, uint64_t workspace_size,
                                           void *t, void const *pos_ids, void const *sin_table,
                                           void const *cos_table, void *stream) {
    (void) workspace;
    (void) workspace_size;
    if (desc == nullptr) return STATUS_BAD_DEVICE;
    auto *d = reinterpret_cast<RoPEDesc *>(desc);
    if (d->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (t == nullptr || pos_ids == nullptr || sin_table == nullptr || cos_table == nullptr) return STATUS_BAD_PARAM;
    if (d->to_dst) return STATUS_BAD_PARAM;// a descriptor of infiniopRoPERearrange
    if (d->seq_len == 0 || d->nhead == 0 || d->dim == 0) return STATUS_SUCCESS;
    DeviceGuard guard(d->device_id);
    return run(d, t, t, pos_ids, sin_table, cos_table, reinterpret_cast<cudaStream_t>(stream));
}

INFINIOP_API infiniopStatus_t infiniopDestroyRoPEDescriptor(infiniopRoPEDescriptor_t desc) {
    if (desc == nullptr) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<RoPEDesc *>(desc);
    return STATUS_SUCCESS;
}

// ---- rotation written to a second view (no counterpart in the reference) ----------------------------------
INFINIOP_API infiniopStatus_t infiniopCreateRoPERearrangeDescriptor(infiniopHandle_t handle,
                                                                    infiniopRoPERearrangeDescriptor_t *desc_ptr,
                                                                    infiniopTensorDescriptor_t dst,
                                                                    infiniopTensorDescriptor_t src,
                                                                    infiniopTensorDescriptor_t pos_ids,
                                                                    infiniopTensorDescriptor_t sin_table,
                                                                    infiniopTensorDescriptor_t cos_table) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (dst == nullptr) return STATUS_BAD_PARAM;
    // `src` passes the checks of the in-place operator; `dst` must be a view of the same shape and type
    infiniopRoPEDescriptor_t made = nullptr;
    const infiniopStatus_t status = infiniopCreateRoPEDescriptor(handle, &made, src, pos_ids, sin_table, cos_table);
    if (status != STATUS_SUCCESS) return status;
    auto *d = reinterpret_cast<RoPEDesc *>(made);
    infiniopStatus_t bad = STATUS_SUCCESS;
    if (dst->ndim != 3 || dst->shape[0] != d->seq_len || dst->shape[1] != d->nhead || dst->shape[2] != d->dim) {
        bad = STATUS_BAD_TENSOR_SHAPE;
    } else if (dst->strides[2] != 1) {
        bad = STATUS_BAD_TENSOR_STRIDES;
    } else if (store_type_of(dst->dt) != d->dt) {
        bad = STATUS_BAD_TENSOR_DTYPE;
    }
    if (bad != STATUS_SUCCESS) {
        delete d;
        return bad;
    }
    d->to_dst = true;
    d->dstride_0 = dst->strides[0];
    d->dstride_1 = dst->strides[1];
    *desc_ptr = reinterpret_cast<infiniopRoPERearrangeDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetRoPERearrangeWorkspaceSize(infiniopRoPERearrangeDescriptor_t desc,
                                                                    uint64_t *size) {
    if (desc == nullptr) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = 0;
    return STATUS_SUCCESS;
}

// `dst` and `src` must not overlap unless they are the same view (then this is infiniopRoPE).
INFINIOP_API infiniopStatus_t infiniopRoPERearrange(infiniopRoPERearrangeDescriptor_t desc, void *workspace,
                                                    uint64_t workspace_size, void *dst, void const *src,
                                                    void const *pos_ids, void const *sin_table,
                                                    void const *cos_table, void *stream) {
    (void) workspace;
    (void) workspace_size;
    if (desc == nullptr) return STATUS_BAD_DEVICE;
    auto *d = reinterpret_cast<RoPEDesc *>(desc);
    if (d->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (dst == nullptr || src == nullptr || pos_ids == nullptr || sin_table == nullptr || cos_table == nullptr) {
        return STATUS_BAD_PARAM;
    }
    if (!d->to_dst) return STATUS_BAD_PARAM;
    if (d->seq_len == 0 || d->nhead == 0 || d->dim == 0) return STATUS_SUCCESS;
    DeviceGuard guard(d->device_id);
    return run(d, dst, src, pos_ids, sin_table, cos_table, reinterpret_cast<cudaStream_t>(stream));
}

INFINIOP_API infiniopStatus_t infiniopDestroyRoPERearrangeDescriptor(infiniopRoPERearrangeDescriptor_t desc) {
    if (desc == nullptr) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<RoPEDesc *>(desc);
    return STATUS_SUCCESS;
}
