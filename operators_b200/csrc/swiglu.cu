// SwiGLU: c = a * silu(b) on 2-D fp16 tensors with independent row strides.
//
// Replaces reference src/ops/swiglu/cuda/swiglu.cu:6-68 and
// src/ops/swiglu/cuda/swiglu_cuda.cc:5-45 behind include/ops/swiglu/swiglu.h.
// Arithmetic follows the reference CPU backend (src/ops/swiglu/cpu/swiglu_cpu.cc:
// 49-73): fp32 silu(b) = b / (1 + exp(-b)), one fp32 multiply by a, and the
// reference's truncating fp32 -> fp16 conversion.  exp(-b) is 2^(-b*log2 e) on
// the special-function unit (relative error ~2^-21 for the |b| that matter) and
// the quotient is b * rcp(d) plus one fused correction step; libm's expf and the
// compiler's IEEE division sequence together cost ~15 % of the achievable
// bandwidth on B200 and change fewer than 1 in 500 truncated outputs (each by
// one fp16 ulp, inside the 1e-3 tolerance).
//
// HBM-bound: 6 bytes move per element.  One CTA of 256 threads per tile of 1024
// vectors (measured on B200: one tile per CTA sustains ~8 % more bandwidth than
// a persistent grid-stride loop); each thread keeps 4 x (a, b) 128-bit streaming
// loads in flight before it computes.  Rows are addressed as flat-vector-index -> (row, column) with a
// multiply-high divider, which keeps arbitrary row strides (the MLP's fused
// gate_up halves: row stride 2*di) on the vector path.  Tensors whose rows are
// not 16-byte aligned take the scalar kernel.
#include "common.cuh"

#include <new>

using namespace b200;

namespace {

struct SwiGLUDesc {
    Device device;
    int device_id;
    int sm_count;
    uint64_t seq_len, di;
    int64_t stride_c, stride_a, stride_b;
    int dt;// kF16, or kBF16 (an extension: bf16 storage, same fp32 arithmetic)
};

__device__ __forceinline__ float swiglu_one(float a, float b) {
    // Very negative b would overflow the exponential to +inf and poison the
    // correction step with inf * 0; any such silu(b) is below 2^-100 and
    // truncates to a signed zero, exactly as with the clamped argument.
    const float e = fast_exp2(fminf(b * -kLog2e, 125.0f));
    const float d = __fadd_rn(1.0f, e);
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    const float q0 = __fmul_rn(b, r);
    const float q = fmaf(fmaf(-q0, d, b), r, q0);
    return __fmul_rn(a, q);
}

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template<int DT>
__global__ void __launch_bounds__(kThreads)
    swiglu_vec8_kernel(uint16_t *c, const uint16_t *a, const uint16_t *b, int64_t stride_c, int64_t stride_a,
                       int64_t stride_b, FastDiv vecs_per_row, uint32_t total_vecs) {
    {
        const uint32_t base = blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
        uint4 va[kUnroll], vb[kUnroll];
        int64_t off_c[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t v = base + u * kThreads;
            if (v < total_vecs) {
                uint32_t row, col;
                vecs_per_row.divmod(v, row, col);
                va[u] = ld_stream(a + (int64_t) row * stride_a + col * 8);
                vb[u] = ld_stream(b + (int64_t) row * stride_b + col * 8);
                off_c[u] = (int64_t) row * stride_c + col * 8;
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t v = base + u * kThreads;
            if (v < total_vecs) {
                const uint32_t *pa = reinterpret_cast<const uint32_t *>(&va[u]);
                const uint32_t *pb = reinterpret_cast<const uint32_t *>(&vb[u]);
                uint4 out;
                uint32_t *po = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float2 fa = unpack2_t<DT>(pa[k]), fb = unpack2_t<DT>(pb[k]);
                    po[k] = pack2_t<DT>(swiglu_one(fa.x, fb.x), swiglu_one(fa.y, fb.y));
                }
                st_stream(c + off_c[u], out);
            }
        }
    }
}

// Any alignment, any row length: one element per thread per step.
template<int DT>
__global__ void __launch_bounds__(kThreads)
    swiglu_scalar_kernel(uint16_t *c, const uint16_t *a, const uint16_t *b, int64_t stride_c, int64_t stride_a,
                         int64_t stride_b, uint64_t di, uint64_t total) {
    for (uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x; i < total; i += (uint64_t) gridDim.x * kThreads) {
        const uint64_t row = i / di, col = i - row * di;
        const float av = load16<DT>(a[(int64_t) row * stride_a + (int64_t) col]);
        const float bv = load16<DT>(b[(int64_t) row * stride_b + (int64_t) col]);
        c[(int64_t) row * stride_c + (int64_t) col] = store16<DT>(swiglu_one(av, bv));
    }
}

}// namespace

INFINIOP_API infiniopStatus_t infiniopCreateSwiGLUDescriptor(infiniopHandle_t handle,
                                                             infiniopSwiGLUDescriptor_t *desc_ptr,
                                                             infiniopTensorDescriptor_t c_desc,
                                                             infiniopTensorDescriptor_t a_desc,
                                                             infiniopTensorDescriptor_t b_desc) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (c_desc == nullptr || a_desc == nullptr || b_desc == nullptr) return STATUS_BAD_PARAM;
    // Same checks, same order, same codes as reference swiglu_cuda.cc:10-36.
    if (c_desc->ndim != 2 || a_desc->ndim != 2 || b_desc->ndim != 2) return STATUS_BAD_TENSOR_SHAPE;
    if (!dt_eq(c_desc->dt, F16) && !dt_eq(c_desc->dt, BF16)) return STATUS_BAD_TENSOR_DTYPE;// bf16: an extension
    if (a_desc->strides[1] != 1 || b_desc->strides[1] != 1 || c_desc->strides[1] != 1) return STATUS_BAD_TENSOR_STRIDES;
    const uint64_t seq_len = c_desc->shape[0], di = c_desc->shape[1];
    if (a_desc->shape[0] != seq_len || a_desc->shape[1] != di || !dt_eq(a_desc->dt, c_desc->dt) ||
        b_desc->shape[0] != seq_len || b_desc->shape[1] != di || !dt_eq(b_desc->dt, c_desc->dt)) {
        return STATUS_BAD_PARAM;
    }
    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow) SwiGLUDesc{DevNvGpu,          h->device_id,       h->sm_count,       seq_len, di,
                                            c_desc->strides[0], a_desc->strides[0], b_desc->strides[0],
                                            store_type_of(c_desc->dt)};
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    *desc_ptr = reinterpret_cast<infiniopSwiGLUDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopSwiGLU(infiniopSwiGLUDescriptor_t desc, void *c, void const *a, void const *b,
                                             void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (c == nullptr || a == nullptr || b == nullptr) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<SwiGLUDesc *>(desc);
    if (d->seq_len == 0 || d->di == 0) return STATUS_SUCCESS;
    DeviceGuard guard(d->device_id);
    auto st = reinterpret_cast<cudaStream_t>(stream);
    auto *cp = reinterpret_cast<uint16_t *>(c);
    auto *ap = reinterpret_cast<const uint16_t *>(a);
    auto *bp = reinterpret_cast<const uint16_t *>(b);

    const bool vec_ok = d->di % 8 == 0 && d->stride_a % 8 == 0 && d->stride_b % 8 == 0 && d->stride_c % 8 == 0 &&
                        aligned16(c) && aligned16(a) && aligned16(b);
    if (vec_ok) {
        const uint64_t vpr = d->di / 8;
        // Row chunks keep the flat vector index inside 32 bits for any tensor size.
        const uint64_t max_vecs = 1ull << 31;
        const uint64_t rows_per_launch = vpr >= max_vecs ? 0 : max_vecs / vpr;
        if (rows_per_launch > 0) {
            for (uint64_t r0 = 0; r0 < d->seq_len; r0 += rows_per_launch) {
                const uint64_t rows = (d->seq_len - r0 < rows_per_launch) ? d->seq_len - r0 : rows_per_launch;
                const uint32_t total = (uint32_t) (rows * vpr);
                const uint32_t tiles = (total + kThreads * kUnroll - 1) / (kThreads * kUnroll);
                auto *kernel = d->dt == kBF16 ? swiglu_vec8_kernel<kBF16> : swiglu_vec8_kernel<kF16>;
                kernel<<<tiles, kThreads, 0, st>>>(cp + (int64_t) r0 * d->stride_c, ap + (int64_t) r0 * d->stride_a,
                                                  bp + (int64_t) r0 * d->stride_b, d->stride_c, d->stride_a, d->stride_b,
                                                  FastDiv((uint32_t) vpr), total);
            }
            return check_launch("swiglu");
        }
    }
    const uint64_t total = d->seq_len * d->di;
    uint64_t blocks = (total + kThreads - 1) / kThreads;
    const uint64_t cap = (uint64_t) d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    auto *scalar = d->dt == kBF16 ? swiglu_scalar_kernel<kBF16> : swiglu_scalar_kernel<kF16>;
    scalar<<<(uint32_t) blocks, kThreads, 0, st>>>(cp, ap, bp, d->stride_c, d->stride_a, d->stride_b, d->di, total);
    return check_launch("swiglu");
}

INFINIOP_API infiniopStatus_t infiniopDestroySwiGLUDescriptor(infiniopSwiGLUDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<SwiGLUDesc *>(desc);
    return STATUS_SUCCESS;
}
