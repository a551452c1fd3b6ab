// Causal softmax, in place on fp16 [.., seq_len, total_seq_len].
//
// Replaces reference src/ops/causal_softmax/cuda/causal_softmax.cu:6-258 and
// src/ops/causal_softmax/cuda/causal_softmax.cc:5-45 behind
// include/ops/causal_softmax/causal_softmax.h.  Semantics follow the CPU backend
// (src/ops/causal_softmax/cpu/causal_softmax_cpu.cc:52-82): row i keeps columns
// j <= total - seq + i, masked columns become exact zeros, the maximum and the
// sum of expf(x - max) are taken over the visible columns in fp32 and each
// output is exp(x - max) / sum narrowed with the reference's truncating
// conversion.  Departures, all far inside the 2e-3 tolerance: the fp32 sum is a
// tree (not sequential), exp is 2^(.) on the special-function unit (relative
// error ~2^-20) and the quotient is e * (1/sum).
//
// HBM-bound: every visible element is read once and every element written
// once; masked tails are never read.  A row lives in registers between the
// three steps (max, exp+sum, scale), owned by one warp or one CTA.
#include "common.cuh"
#include "row_ring.cuh"
#include "fastdiv.h"

#include <new>

using namespace b200;

namespace {

struct CausalSoftmaxDesc {
    Device device;
    int device_id;
    int sm_count;
    uint64_t batch, seq_len, total;
    int64_t stride_b, stride_i;
    int dt;// kF16, or kBF16 (an extension: bf16 storage, same fp32 arithmetic)
};

// Number of visible columns of query row i (at least 1: column 0 always is).
__device__ __forceinline__ uint64_t visible_cols(uint64_t i, uint64_t seq_len, uint64_t total) {
    const uint64_t last = total - seq_len + i;// wraps like the reference when seq_len > total
    return last >= total - 1 ? total : last + 1;
}

// The row stays in registers as the PACKED fp16 it was loaded as (4 registers
// per vector), which keeps the register count low enough for 12-16 resident
// rows per SM, i.e. ~100 KB of loads in flight.  The maximum is taken on the
// packed halves; the exponential is evaluated twice (once for the sum, once for
// the output) as the CPU code does, which costs less than holding the row in
// fp32 would cost in occupancy.  (The compiler is free to keep the first
// evaluation instead; measured, that is the faster of the two on B200.)
//
// Who owns a row: one warp, one CTA, or one thread-block cluster of 2, 4 or 8 CTAs whose maxima and sums meet
// over distributed shared memory (rows of more than 32 Ki columns).
enum RowOwner { WARP_ROW = 0, CTA_ROW = 1, CLUSTER_ROW = 2 };

// packed maximum of two 16-bit pairs
template<int DT>
__device__ __forceinline__ uint32_t max2_packed(uint32_t a, uint32_t b) {
    uint32_t r;
    if (DT == kBF16) asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    else asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

template<int VPT, int OWNER, int DT>
__device__ __forceinline__ void causal_softmax_regs_body(uint16_t *y, uint64_t rows, uint64_t seq_len, uint64_t total,
                                                         uint32_t vecs, int64_t stride_b, int64_t stride_i, FastDiv seq_div) {
    __shared__ float red_m[32], red_s[32];// one slot array per reduction of a row: one barrier each
    __shared__ float part_m, part_s;      // this CTA's maximum and sum, read by the whole cluster
    const int lane = threadIdx.x & 31;
    const uint32_t cl = OWNER == CLUSTER_ROW ? cluster_size() : 1;
    const uint32_t group = OWNER == WARP_ROW ? 32 : blockDim.x * cl;
    const uint32_t t = OWNER == WARP_ROW ? lane : (OWNER == CLUSTER_ROW ? cluster_rank() * blockDim.x : 0) + threadIdx.x;
    const uint64_t rows_per_cta = OWNER == WARP_ROW ? (blockDim.x >> 5) : 1;
    const uint64_t row0 = OWNER == WARP_ROW ? (uint64_t) blockIdx.x * rows_per_cta + (threadIdx.x >> 5)
                                            : (uint64_t) (blockIdx.x / cl);
    const uint64_t row_step = OWNER == WARP_ROW ? (uint64_t) gridDim.x * rows_per_cta : (uint64_t) (gridDim.x / cl);
    constexpr uint32_t kNegInf1 = DT == kBF16 ? 0xFF80u : 0xFC00u;// -inf
    constexpr uint32_t kNegInf2 = kNegInf1 * 0x00010001u;          // two of them

    for (uint64_t row = row0; row < rows; row += row_step) {
        uint64_t b, i;
        if (rows <= 0xFFFFFFFFull) {// the usual case: one multiply-high instead of a 64-bit division
            uint32_t q, r;
            seq_div.divmod((uint32_t) row, q, r);
            b = q, i = r;
        } else {
            b = row / seq_len, i = row - b * seq_len;
        }
        uint16_t *yr = y + (int64_t) b * stride_b + (int64_t) i * stride_i;
        const uint32_t vis = (uint32_t) visible_cols(i, seq_len, total);

        uint4 raw[VPT];
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            if (j < vecs && j * 8 < vis) raw[u] = ld_stream(yr + (uint64_t) j * 8);
            else raw[u] = make_uint4(kNegInf2, kNegInf2, kNegInf2, kNegInf2);// masked: exp -> 0, output 0
        }
        uint32_t m2 = kNegInf2;
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            uint32_t *p = reinterpret_cast<uint32_t *>(&raw[u]);
            if (j * 8 < vis && j * 8 + 8 > vis) {// the one vector that straddles the mask boundary
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (j * 8 + 2 * k >= vis) p[k] = (p[k] & 0xFFFF0000u) | kNegInf1;
                    if (j * 8 + 2 * k + 1 >= vis) p[k] = (p[k] & 0x0000FFFFu) | (kNegInf1 << 16);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) m2 = max2_packed<DT>(m2, p[k]);
        }
        const float2 mm = unpack2_t<DT>(m2);
        float m = fmaxf(mm.x, mm.y);
        if (OWNER == CLUSTER_ROW) m = cluster_reduce<true>(m, red_m, &part_m, cl);
        else m = OWNER == CTA_ROW ? cta_reduce_alt<true>(m, red_m) : warp_max(m);
        // exp(x - m) = 2^(x*log2e - m*log2e); the rounding of m*log2e is common to
        // the whole row and cancels in the quotient.
        const float mk = -m * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t *p = reinterpret_cast<const uint32_t *>(&raw[u]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = unpack2_t<DT>(p[k]);
                s += fast_exp2(fmaf(f.x, kLog2e, mk));
                s += fast_exp2(fmaf(f.y, kLog2e, mk));
            }
        }
        if (OWNER == CLUSTER_ROW) s = cluster_reduce<false>(s, red_s, &part_s, cl);
        else s = OWNER == CTA_ROW ? cta_reduce_alt<false>(s, red_s) : warp_sum(s);
        const float r = __frcp_rn(s);
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            if (j < vecs) {
                const uint32_t *p = reinterpret_cast<const uint32_t *>(&raw[u]);
                uint4 out;
                uint32_t *po = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = unpack2_t<DT>(p[k]);
                    const float q0 = __fmul_rn(fast_exp2(fmaf(f.x, kLog2e, mk)), r);
                    const float q1 = __fmul_rn(fast_exp2(fmaf(f.y, kLog2e, mk)), r);
                    // quotients lie in [0, 1]: the packed truncating convert needs no range check
                    if (DT == kBF16) po[k] = (__float_as_uint(q0) >> 16) | (__float_as_uint(q1) & 0xFFFF0000u);
                    else asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(po[k]) : "f"(q1), "f"(q0));
                }
                st_stream(yr + (uint64_t) j * 8, out);
            }
        }
        // no CTA may leave (or start its next row) while a neighbour still reads its maximum or sum
        if (OWNER == CLUSTER_ROW) cluster_sync_all();
    }
}

// Two kernels around the one body: without a launch bound for up to 512 threads (the compiler's own register
// choice), bounded to 1024 threads (64 registers) for the forms launched with more.
template<int VPT, int OWNER, int MAXT, int DT>
__global__ void causal_softmax_regs_kernel(uint16_t *y, uint64_t rows, uint64_t seq_len, uint64_t total, uint32_t vecs,
                                           int64_t stride_b, int64_t stride_i, FastDiv seq_div) {
    static_assert(MAXT <= 512, "launches of more than 512 threads use causal_softmax_regs_kernel_1024");
    causal_softmax_regs_body<VPT, OWNER, DT>(y, rows, seq_len, total, vecs, stride_b, stride_i, seq_div);
}
template<int VPT, int OWNER, int DT>
__global__ void __launch_bounds__(1024)
    causal_softmax_regs_kernel_1024(uint16_t *y, uint64_t rows, uint64_t seq_len, uint64_t total, uint32_t vecs,
                                    int64_t stride_b, int64_t stride_i, FastDiv seq_div) {
    causal_softmax_regs_body<VPT, OWNER, DT>(y, rows, seq_len, total, vecs, stride_b, stride_i, seq_div);
}

// Rows of 32 Ki columns and more, many of them: the shared-memory ring of row_ring.cuh.
template<int DT>
__global__ void __launch_bounds__(ring::kThreads, 1)
    causal_softmax_ring_kernel(uint16_t *y, uint64_t rows, uint64_t seq_len, uint64_t total, uint32_t vecs,
                               int64_t stride_b, int64_t stride_i, ring::Plan plan) {
    ring::causal_softmax_ring_body<DT>(y, rows, seq_len, total, vecs, stride_b, stride_i, plan);
}

// Any alignment, any column stride, any row length: one CTA per row, three
// passes (max / sum / write), the later ones served by L2.
template<int DT>
__global__ void causal_softmax_generic_kernel(uint16_t *y, uint64_t rows, uint64_t seq_len, uint64_t total,
                                              int64_t stride_b, int64_t stride_i) {
    __shared__ float red[32];
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint64_t b = row / seq_len, i = row - b * seq_len;
        uint16_t *yr = y + (int64_t) b * stride_b + (int64_t) i * stride_i;
        const uint64_t vis = visible_cols(i, seq_len, total);
        float m = -INFINITY;
        for (uint64_t j = threadIdx.x; j < vis; j += blockDim.x) m = fmaxf(m, load16<DT>(yr[j]));
        m = cta_reduce<true>(m, red);
        float s = 0.f;
        for (uint64_t j = threadIdx.x; j < vis; j += blockDim.x) s += expf(__fsub_rn(load16<DT>(yr[j]), m));
        s = cta_reduce<false>(s, red);
        const float r = __frcp_rn(s);
        for (uint64_t j = threadIdx.x; j < total; j += blockDim.x) {
            uint16_t out = 0;
            if (j < vis) {
                const float e = expf(__fsub_rn(load16<DT>(yr[j]), m));
                const float q0 = __fmul_rn(e, r);
                out = store16<DT>(fmaf(fmaf(-q0, s, e), r, q0));
            }
            yr[j] = out;
        }
        __syncthreads();
    }
}

// false: no register-resident kernel fits this shape (the caller takes the three-pass kernel)
template<int VPT, int DT>
bool launch_regs(const CausalSoftmaxDesc *d, bool cta_row, uint32_t threads, uint32_t cl, uint32_t vecs, uint16_t *y,
                 cudaStream_t st) {
    const uint64_t rows = d->batch * d->seq_len;
    const FastDiv seq_div(d->seq_len <= 0xFFFFFFFFull && d->seq_len > 0 ? (uint32_t) d->seq_len : 1u);
    if (cta_row) {
        const uint64_t cap = 0x7FFFFFFFull / cl;// one CTA (cluster) per row; rows beyond that loop
        const uint32_t grid = (uint32_t) (rows < cap ? rows : cap) * cl;
        if (cl > 1) {
            if constexpr (VPT == 4) {// clusters always hold four vectors per thread
                launch_cluster(causal_softmax_regs_kernel_1024<4, CLUSTER_ROW, DT>, grid, threads, cl, st, y, rows,
                               d->seq_len, d->total, vecs, d->stride_b, d->stride_i, seq_div);
                return true;
            }
            return false;
        }
        if (threads <= 512 && fits_register_file<causal_softmax_regs_kernel<VPT, CTA_ROW, 512, DT>>(threads)) {
            causal_softmax_regs_kernel<VPT, CTA_ROW, 512, DT>
                <<<grid, threads, 0, st>>>(y, rows, d->seq_len, d->total, vecs, d->stride_b, d->stride_i, seq_div);
            return true;
        }
        if constexpr (VPT <= 4) {// bounded to 64 registers: any block size
            causal_softmax_regs_kernel_1024<VPT, CTA_ROW, DT>
                <<<grid, threads, 0, st>>>(y, rows, d->seq_len, d->total, vecs, d->stride_b, d->stride_i, seq_div);
            return true;
        }
        return false;
    }
    const uint64_t ctas = (rows + 7) / 8;
    const uint64_t cap = 0x7FFFFFFFull;
    const uint32_t grid = (uint32_t) (ctas < cap ? ctas : cap);
    if (!fits_register_file<causal_softmax_regs_kernel<VPT, WARP_ROW, 256, DT>>(256)) return false;
    causal_softmax_regs_kernel<VPT, WARP_ROW, 256, DT>
        <<<grid, 256, 0, st>>>(y, rows, d->seq_len, d->total, vecs, d->stride_b, d->stride_i, seq_div);
    return true;
}

}// namespace

namespace b200 {
unsigned long long causal_softmax_ring_timeouts_read() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, ring::g_row_ring_timeouts, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return ~0ull;
    }
    return v;
}
}// namespace b200

INFINIOP_API infiniopStatus_t infiniopCreateCausalSoftmaxDescriptor(infiniopHandle_t handle,
                                                                    infiniopCausalSoftmaxDescriptor_t *desc_ptr,
                                                                    infiniopTensorDescriptor_t y) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (y == nullptr) return STATUS_BAD_PARAM;
    // Checks, order and codes of reference causal_softmax.cc:8-24.
    const uint64_t ndim = y->ndim;
    if (ndim != 2 && ndim != 3) return STATUS_BAD_TENSOR_SHAPE;
    if (!dt_eq(y->dt, F16) && !dt_eq(y->dt, BF16)) return STATUS_BAD_TENSOR_DTYPE;// bf16: an extension
    if (y->strides[ndim - 1] != 1) return STATUS_BAD_TENSOR_STRIDES;
    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow) CausalSoftmaxDesc{DevNvGpu,
                                                   h->device_id,
                                                   h->sm_count,
                                                   ndim == 3 ? y->shape[0] : 1,
                                                   y->shape[ndim - 2],
                                                   y->shape[ndim - 1],
                                                   ndim == 3 ? y->strides[0] : 0,
                                                   y->strides[ndim - 2],
                                                   store_type_of(y->dt)};
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

    // rows of up to 8 CTAs x 1024 threads x 4 vectors stay in registers
    const bool vec_ok = d->total % 8 == 0 && d->total / 8 <= 32768 && d->stride_i % 8 == 0 && d->stride_b % 8 == 0 &&
                        aligned16(data);
    if (vec_ok) {
        const uint32_t vecs = (uint32_t) (d->total / 8);
        const bool big = rows * (uint64_t) vecs >= (1u << 20);
        // The shared-memory ring never beat the register kernels here (32768 columns: 175 against 148 us, 65536: equal,
        // longer rows slower): it runs only when infiniopExtSelectKernel(long rows, 2) asks for it (4096 columns and more).
        const int ring_choice = kernel_choice(kFamilyLongRows);
        if (ring_choice == 2 && vecs >= 512) {
            ring::Plan plan;
            if (ring::make_plan(plan, vecs, rows, d->sm_count)) {
                auto *kernel = d->dt == kBF16 ? causal_softmax_ring_kernel<kBF16> : causal_softmax_ring_kernel<kF16>;
                if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) plan.smem_bytes) ==
                    cudaSuccess) {
                    if (plan.cl > 1) {
                        launch_cluster_smem(kernel, plan.grid, ring::kThreads, plan.cl, plan.smem_bytes, st, y, rows,
                                            d->seq_len, d->total, vecs, d->stride_b, d->stride_i, plan);
                    } else {
                        kernel<<<plan.grid, ring::kThreads, plan.smem_bytes, st>>>(y, rows, d->seq_len, d->total, vecs,
                                                                                  d->stride_b, d->stride_i, plan);
                    }
                    return check_launch("causal_softmax (ring)");
                }
                cudaGetLastError();
            }
        }
        int vpt;
        bool cta_row;
        uint32_t threads = 256, cl = 1;
        if (big && vecs <= 256) {
            cta_row = false;
            const uint32_t need = (vecs + 31) / 32;
            vpt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
        } else {
            cta_row = true;
            // measured at [32,512,4096]: 4 vectors per thread (128 threads per 4096-column
            // row) 50 us, 8 per thread 52 us, 2 per thread 63 us
            // rows of 16384 columns and more: 8 per thread (0.73 against 0.67 of the copy bandwidth at
            // [16, 512, 16384], 0.55 against 0.50 at [8, 512, 32768]; no difference at 8192 columns).
            // Rows of more than 4096 vectors are spread over a cluster of 2, 4 or 8 CTAs.
            const RowLaunch shape = row_launch_shape(vecs, big ? (vecs >= 2048 ? 8 : 4) : 1);
            vpt = shape.vpt, threads = shape.threads, cl = shape.cl;
        }
        bool launched;
        if (d->dt == kBF16) {
            launched = vpt == 1 ? launch_regs<1, kBF16>(d, cta_row, threads, cl, vecs, y, st)
                     : vpt == 2 ? launch_regs<2, kBF16>(d, cta_row, threads, cl, vecs, y, st)
                     : vpt == 4 ? launch_regs<4, kBF16>(d, cta_row, threads, cl, vecs, y, st)
                                : launch_regs<8, kBF16>(d, cta_row, threads, cl, vecs, y, st);
        } else {
            launched = vpt == 1 ? launch_regs<1, kF16>(d, cta_row, threads, cl, vecs, y, st)
                     : vpt == 2 ? launch_regs<2, kF16>(d, cta_row, threads, cl, vecs, y, st)
                     : vpt == 4 ? launch_regs<4, kF16>(d, cta_row, threads, cl, vecs, y, st)
                                : launch_regs<8, kF16>(d, cta_row, threads, cl, vecs, y, st);
        }
        if (launched) return check_launch("causal_softmax");
    }
    const uint64_t cap = (uint64_t) d->sm_count * 8;
    const uint32_t grid = (uint32_t) (rows < cap ? rows : cap);
    auto *generic = d->dt == kBF16 ? causal_softmax_generic_kernel<kBF16> : causal_softmax_generic_kernel<kF16>;
    generic<<<grid, 256, 0, st>>>(y, rows, d->seq_len, d->total, d->stride_b, d->stride_i);
    return check_launch("causal_softmax");
}

INFINIOP_API infiniopStatus_t infiniopDestroyCausalSoftmaxDescriptor(infiniopCausalSoftmaxDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<CausalSoftmaxDesc *>(desc);
    return STATUS_SUCCESS;
}
