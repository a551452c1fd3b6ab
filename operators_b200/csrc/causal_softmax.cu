// Causal softmax, in place on fp16 [.., seq_len, total_seq_len].
//
// Replaces reference src/ops/causal_softmax/cuda/causal_softmax.cu:6-258 and
// src/ops/causal_softmax/cuda/causal_softmax.cc:5-45 behind
// include/ops/causal_softmax/causal_softmax.h.  Semantics follow the CPU backend
// (src/ops/causal_softmax/cpu/causal_softmax_cpu.cc:52-82): row i keeps columns
// j <= total - seq + i, masked columns become exact zeros, the maximum and the
// sum of expf(x - max) are taken over the visible columns in fp32 and each
// output is expf(x - max) / sum narrowed with the reference's truncating
// conversion.  Departures: the fp32 sum is a tree (not sequential) and the
// quotient is formed as e * (1/sum) with one fused correction step, which
// returns the correctly rounded quotient in all but rare half-ulp cases.
//
// HBM-bound: every visible element is read once and every element written
// once; masked tails are never read.  A row lives in registers as fp32 between
// the three steps (max, exp+sum, scale), owned by one warp or one CTA.
#include "common.cuh"

#include <new>

using namespace b200;

namespace {

struct CausalSoftmaxDesc {
    Device device;
    int device_id;
    int sm_count;
    uint64_t batch, seq_len, total;
    int64_t stride_b, stride_i;
};

// Number of visible columns of query row i (at least 1: column 0 always is).
__device__ __forceinline__ uint64_t visible_cols(uint64_t i, uint64_t seq_len, uint64_t total) {
    const uint64_t last = total - seq_len + i;// wraps like the reference when seq_len > total
    return last >= total - 1 ? total : last + 1;
}

template<int VPT, bool CTA_ROW>
__global__ void causal_softmax_regs_kernel(uint16_t *y, uint64_t rows, uint64_t seq_len, uint64_t total,
                                           uint32_t vecs, int64_t stride_b, int64_t stride_i) {
    __shared__ float red[32];
    const int lane = threadIdx.x & 31;
    const uint32_t group = CTA_ROW ? blockDim.x : 32;
    const uint32_t t = CTA_ROW ? threadIdx.x : lane;
    const uint64_t rows_per_cta = CTA_ROW ? 1 : (blockDim.x >> 5);
    const uint64_t row0 = (uint64_t) blockIdx.x * rows_per_cta + (CTA_ROW ? 0 : (threadIdx.x >> 5));
    const uint64_t row_step = (uint64_t) gridDim.x * rows_per_cta;

    for (uint64_t row = row0; row < rows; row += row_step) {
        const uint64_t b = row / seq_len, i = row - b * seq_len;
        uint16_t *yr = y + (int64_t) b * stride_b + (int64_t) i * stride_i;
        const uint32_t vis = (uint32_t) visible_cols(i, seq_len, total);

        float f[VPT][8];
        uint4 raw[VPT];
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            if (j < vecs && j * 8 < vis) raw[u] = ld_stream(yr + (uint64_t) j * 8);
        }
        float m = -INFINITY;
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            const bool loaded = j < vecs && j * 8 < vis;
            const uint32_t *p = reinterpret_cast<const uint32_t *>(&raw[u]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 v = loaded ? unpack2(p[k]) : make_float2(-INFINITY, -INFINITY);
                if (j * 8 + 2 * k >= vis) v.x = -INFINITY;
                if (j * 8 + 2 * k + 1 >= vis) v.y = -INFINITY;
                f[u][2 * k] = v.x;
                f[u][2 * k + 1] = v.y;
                m = fmaxf(m, fmaxf(v.x, v.y));
            }
        }
        m = CTA_ROW ? cta_reduce<true>(m, red) : warp_max(m);
        float s = 0.f;
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                // masked slots hold -inf: expf(-inf - m) = 0 contributes nothing
                f[u][e] = expf(__fsub_rn(f[u][e], m));
                s += f[u][e];
            }
        }
        s = CTA_ROW ? cta_reduce<false>(s, red) : warp_sum(s);
        const float r = __frcp_rn(s);
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            if (j < vecs) {
                uint4 out;
                uint32_t *po = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float q[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float e = f[u][2 * k + h];
                        const float q0 = __fmul_rn(e, r);
                        q[h] = fmaf(fmaf(-q0, s, e), r, q0);
                    }
                    po[k] = pack2_ref(q[0], q[1]);
                }
                st_stream(yr + (uint64_t) j * 8, out);
            }
        }
    }
}

// Any alignment, any column stride, any row length: one CTA per row, three
// passes (max / sum / write), the later ones served by L2.
__global__ void causal_softmax_generic_kernel(uint16_t *y, uint64_t rows, uint64_t seq_len, uint64_t total,
                                              int64_t stride_b, int64_t stride_i) {
    __shared__ float red[32];
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint64_t b = row / seq_len, i = row - b * seq_len;
        uint16_t *yr = y + (int64_t) b * stride_b + (int64_t) i * stride_i;
        const uint64_t vis = visible_cols(i, seq_len, total);
        float m = -INFINITY;
        for (uint64_t j = threadIdx.x; j < vis; j += blockDim.x) m = fmaxf(m, f16_to_f32(yr[j]));
        m = cta_reduce<true>(m, red);
        float s = 0.f;
        for (uint64_t j = threadIdx.x; j < vis; j += blockDim.x) s += expf(__fsub_rn(f16_to_f32(yr[j]), m));
        s = cta_reduce<false>(s, red);
        const float r = __frcp_rn(s);
        for (uint64_t j = threadIdx.x; j < total; j += blockDim.x) {
            uint16_t out = 0;
            if (j < vis) {
                const float e = expf(__fsub_rn(f16_to_f32(yr[j]), m));
                const float q0 = __fmul_rn(e, r);
                out = f32_to_f16_ref(fmaf(fmaf(-q0, s, e), r, q0));
            }
            yr[j] = out;
        }
        __syncthreads();
    }
}

template<int VPT>
void launch_regs(const CausalSoftmaxDesc *d, bool cta_row, uint32_t threads, uint32_t vecs, uint16_t *y,
                 cudaStream_t st) {
    const uint64_t rows = d->batch * d->seq_len;
    if (cta_row) {
        const uint64_t cap = 0x7FFFFFFFull;// one CTA per row; rows beyond 2^31 loop
        const uint32_t grid = (uint32_t) (rows < cap ? rows : cap);
        causal_softmax_regs_kernel<VPT, true>
            <<<grid, threads, 0, st>>>(y, rows, d->seq_len, d->total, vecs, d->stride_b, d->stride_i);
    } else {
        const uint64_t ctas = (rows + 7) / 8;
        const uint64_t cap = 0x7FFFFFFFull;
        const uint32_t grid = (uint32_t) (ctas < cap ? ctas : cap);
        causal_softmax_regs_kernel<VPT, false>
            <<<grid, 256, 0, st>>>(y, rows, d->seq_len, d->total, vecs, d->stride_b, d->stride_i);
    }
}

}// namespace

INFINIOP_API infiniopStatus_t infiniopCreateCausalSoftmaxDescriptor(infiniopHandle_t handle,
                                                                    infiniopCausalSoftmaxDescriptor_t *desc_ptr,
                                                                    infiniopTensorDescriptor_t y) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (y == nullptr) return STATUS_BAD_PARAM;
    // Checks, order and codes of reference causal_softmax.cc:8-24.
    const uint64_t ndim = y->ndim;
    if (ndim != 2 && ndim != 3) return STATUS_BAD_TENSOR_SHAPE;
    if (!dt_eq(y->dt, F16)) return STATUS_BAD_TENSOR_DTYPE;
    if (y->strides[ndim - 1] != 1) return STATUS_BAD_TENSOR_STRIDES;
    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow) CausalSoftmaxDesc{DevNvGpu,
                                                   h->device_id,
                                                   h->sm_count,
                                                   ndim == 3 ? y->shape[0] : 1,
                                                   y->shape[ndim - 2],
                                                   y->shape[ndim - 1],
                                                   ndim == 3 ? y->strides[0] : 0,
                                                   y->strides[ndim - 2]};
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    *desc_ptr = reinterpret_cast<infiniopCausalSoftmaxDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetCausalSoftmaxWorkspaceSize(infiniopCausalSoftmaxDescriptor_t desc,
                                                                    uint64_t *size) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = 0;
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopCausalSoftmax(infiniopCausalSoftmaxDescriptor_t desc, void *workspace,
                                                    uint64_t workspace_size, void *data, void *stream) {
    (void) workspace;
    (void) workspace_size;
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (data == nullptr) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<CausalSoftmaxDesc *>(desc);
    const uint64_t rows = d->batch * d->seq_len;
    if (rows == 0 || d->total == 0) return STATUS_SUCCESS;
    DeviceGuard guard(d->device_id);
    auto st = reinterpret_cast<cudaStream_t>(stream);
    auto *y = reinterpret_cast<uint16_t *>(data);

    const bool vec_ok = d->total % 8 == 0 && d->total / 8 <= 8192 && d->stride_i % 8 == 0 && d->stride_b % 8 == 0 &&
                        aligned16(data);
    if (vec_ok) {
        const uint32_t vecs = (uint32_t) (d->total / 8);
        const bool big = rows * (uint64_t) vecs >= (1u << 20);
        int vpt;
        bool cta_row;
        uint32_t threads = 256;
        if (big && vecs <= 128) {
            cta_row = false;
            const uint32_t need = (vecs + 31) / 32;
            vpt = need <= 1 ? 1 : need <= 2 ? 2 : 4;
        } else {
            cta_row = true;
            const uint32_t min_vpt = (vecs + 1023) / 1024;
            uint32_t want = big ? 4 : min_vpt;
            if (want < min_vpt) want = min_vpt;
            vpt = want <= 1 ? 1 : want <= 2 ? 2 : want <= 4 ? 4 : 8;
            threads = ((vecs + vpt - 1) / vpt + 31) / 32 * 32;
        }
        switch (vpt) {
            case 1: launch_regs<1>(d, cta_row, threads, vecs, y, st); break;
            case 2: launch_regs<2>(d, cta_row, threads, vecs, y, st); break;
            case 4: launch_regs<4>(d, cta_row, threads, vecs, y, st); break;
            default: launch_regs<8>(d, cta_row, threads, vecs, y, st); break;
        }
        return check_launch("causal_softmax");
    }
    const uint64_t cap = (uint64_t) d->sm_count * 8;
    const uint32_t grid = (uint32_t) (rows < cap ? rows : cap);
    causal_softmax_generic_kernel<<<grid, 256, 0, st>>>(y, rows, d->seq_len, d->total, d->stride_b, d->stride_i);
    return check_launch("causal_softmax");
}

INFINIOP_API infiniopStatus_t infiniopDestroyCausalSoftmaxDescriptor(infiniopCausalSoftmaxDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<CausalSoftmaxDesc *>(desc);
    return STATUS_SUCCESS;
}
