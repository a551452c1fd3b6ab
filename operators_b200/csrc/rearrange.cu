// Rearrange: dst[i0, .., i_{n-1}] = src[i0, .., i_{n-1}] between two views of the
// same shape and element type whose innermost stride is 1 and whose other
// strides are arbitrary (the copy on both sides of attention: K/V rows into the
// cache at their positions, q made contiguous, the output permuted back).
//
// Replaces reference src/ops/rearrange/cuda/rearrange.cu:4-76 and
// src/ops/rearrange/cuda/rearrange.cc:6-68 behind
// include/ops/rearrange/rearrange.h.  Result = the CPU backend's
// (src/ops/rearrange/cpu/rearrange_cpu.cc:79-100: one memcpy per innermost row),
// byte for byte; bytes are moved, never interpreted, so every DataLayout works.
// Wider than the reference: its nv-gpu code stops at 3 dimensions
// (rearrange.cc:58-59) and its CPU code wants the leading dimensions of longer
// shapes to be mergeable (rearrange_cpu.cc:45-52); here any shape of up to 8
// dimensions with any outer strides is served.  Overlapping dst and src are
// undefined, as for the reference's memcpy.
//
// HBM-bound, two streams.  Neighbouring dimensions that are dense in both
// views are merged on the host; the unit of work is the widest power of two
// (<= 16 bytes) that divides the row length, every stride and both base
// addresses; a flat unit index is split into (row, unit in row) and the row
// into its coordinates with multiply-high dividers passed by value.  One tile
// of kUnroll units per thread per CTA.
#include "common.cuh"
#include "fastdiv.h"

#include <new>

using namespace b200;

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kMaxDims = 8;

struct RowDims {
    int nouter;                 // merged outer dimensions (row coordinates), innermost of them last
    FastDiv div[kMaxDims];      // extent of each outer dimension
    int64_t ds[kMaxDims];       // dst stride in bytes
    int64_t ss[kMaxDims];       // src stride in bytes
};

struct RearrangeDesc {
    Device device;
    int device_id;
    uint32_t elem_size;
    uint64_t row_bytes;         // bytes of one (merged) innermost row
    uint64_t rows;
    int gcd_shift;              // log2 of what divides row_bytes and all strides, at most 4
    RowDims dims;
};

template<int UNIT>
struct UnitType;
template<> struct UnitType<16> { using T = uint4; };
template<> struct UnitType<8> { using T = uint2; };
template<> struct UnitType<4> { using T = uint32_t; };
template<> struct UnitType<2> { using T = uint16_t; };
template<> struct UnitType<1> { using T = uint8_t; };

// units_per_row = row_bytes / UNIT; total = rows * units_per_row < 2^32 * UNIT is split over blockIdx.
template<int UNIT>
__global__ void __launch_bounds__(kThreads) rearrange_kernel(uint8_t *dst, const uint8_t *src, uint64_t total,
                                                             FastDiv units_per_row, RowDims dims) {
    using T = typename UnitType<UNIT>::T;
    const uint64_t tile0 = (uint64_t) blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
    T v[kUnroll];
    int64_t doff[kUnroll];
    bool live[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const uint64_t i = tile0 + (uint64_t) u * kThreads;
        live[u] = i < total;
        doff[u] = 0;
        if (live[u]) {
            uint32_t row, col;
            units_per_row.divmod((uint32_t) i, row, col);
            int64_t so = (int64_t) col * UNIT, dof = so;
            for (int d = dims.nouter - 1; d >= 0; --d) {
                uint32_t q, c;
                dims.div[d].divmod(row, q, c);
                so += (int64_t) c * dims.ss[d];
                dof += (int64_t) c * dims.ds[d];
                row = q;
            }
            doff[u] = dof;
            if (UNIT == 16) *reinterpret_cast<uint4 *>(&v[u]) = ld_stream(src + so);
            else v[u] = *reinterpret_cast<const T *>(src + so);
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        if (live[u]) {
            if (UNIT == 16) st_stream(dst + doff[u], *reinterpret_cast<const uint4 *>(&v[u]));
            else *reinterpret_cast<T *>(dst + doff[u]) = v[u];
        }
    }
}

template<int UNIT>
infiniopStatus_t launch(const RearrangeDesc *d, void *dst, const void *src, cudaStream_t st) {
    const uint64_t upr = d->row_bytes / UNIT;
    const uint64_t total = d->rows * upr;
    const uint64_t per_cta = (uint64_t) kThreads * kUnroll;
    const uint64_t ctas = (total + per_cta - 1) / per_cta;
    if (total > 0xFFFFFFFFull || ctas > 0x7FFFFFFFull) return STATUS_BAD_TENSOR_SHAPE;// more than 2^32 units in one call
    rearrange_kernel<UNIT><<<(uint32_t) ctas, kThreads, 0, st>>>(reinterpret_cast<uint8_t *>(dst),
                                                                 reinterpret_cast<const uint8_t *>(src), total,
                                                                 FastDiv((uint32_t) upr), d->dims);
    return check_launch("rearrange");
}

}// namespace

INFINIOP_API infiniopStatus_t infiniopCreateRearrangeDescriptor(infiniopHandle_t handle,
                                                                infiniopRearrangeDescriptor_t *desc_ptr,
                                                                infiniopTensorDescriptor_t dst,
                                                                infiniopTensorDescriptor_t src) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (dst == nullptr || src == nullptr) return STATUS_BAD_PARAM;
    // checks, order and codes of reference rearrange.cc:10-26
    if (!dt_eq(dst->dt, src->dt)) return STATUS_BAD_TENSOR_DTYPE;
    const uint64_t ndim = dst->ndim;
    if (src->ndim != ndim || ndim == 0) return STATUS_BAD_TENSOR_SHAPE;
    for (uint64_t i = 0; i < ndim; ++i) {
        if (dst->shape[i] != src->shape[i]) return STATUS_BAD_TENSOR_SHAPE;
    }
    if (dst->strides[ndim - 1] != 1 || src->strides[ndim - 1] != 1) return STATUS_BAD_TENSOR_STRIDES;
    const uint32_t esz = dst->dt.size;
    if (esz == 0) return STATUS_BAD_TENSOR_DTYPE;

    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow) RearrangeDesc{};
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    d->device = DevNvGpu;
    d->device_id = h->device_id;
    d->elem_size = esz;

    // Innermost row, grown over every outer dimension that is dense behind it in BOTH views; then the
    // remaining outer dimensions, neighbours merged where one steps exactly over the other in both views.
    uint64_t row_elems = dst->shape[ndim - 1];
    int64_t top = (int64_t) ndim - 2;
    while (top >= 0 && dst->strides[top] == (int64_t) row_elems && src->strides[top] == (int64_t) row_elems) {
        row_elems *= dst->shape[top];
        --top;
    }
    uint64_t shp[kMaxDims];
    int64_t ds[kMaxDims], ss[kMaxDims];
    int n = 0;
    bool empty = row_elems == 0;
    for (int64_t i = 0; i <= top; ++i) {
        const uint64_t e = dst->shape[i];
        if (e == 0) empty = true;
        if (e == 1) continue;
        if (n > 0 && ds[n - 1] == (int64_t) e * dst->strides[i] && ss[n - 1] == (int64_t) e * src->strides[i]) {
            shp[n - 1] *= e;// the previous (outer) dimension steps exactly over this one
            ds[n - 1] = dst->strides[i];
            ss[n - 1] = src->strides[i];
            continue;
        }
        if (n == kMaxDims) {
            delete d;
            return STATUS_BAD_TENSOR_SHAPE;
        }
        shp[n] = e, ds[n] = dst->strides[i], ss[n] = src->strides[i];
        ++n;
    }
    uint64_t rows = 1;
    uint64_t common = row_elems * esz;// bits that row length and every stride have in common
    for (int i = 0; i < n; ++i) {
        if (shp[i] > 0xFFFFFFFFull) {
            delete d;
            return STATUS_BAD_TENSOR_SHAPE;
        }
        rows *= shp[i];
        d->dims.div[i] = FastDiv((uint32_t) shp[i]);
        d->dims.ds[i] = ds[i] * (int64_t) esz;
        d->dims.ss[i] = ss[i] * (int64_t) esz;
        common |= (uint64_t) (ds[i] < 0 ? -ds[i] : ds[i]) * esz | (uint64_t) (ss[i] < 0 ? -ss[i] : ss[i]) * esz;
    }
    d->dims.nouter = n;
    d->row_bytes = row_elems * esz;
    d->rows = empty ? 0 : rows;
    int shift = 0;
    while (shift < 4 && common != 0 && (common & (1ull << shift)) == 0) ++shift;
    d->gcd_shift = common == 0 ? 0 : shift;
    *desc_ptr = reinterpret_cast<infiniopRearrangeDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopRearrange(infiniopRearrangeDescriptor_t desc, void *dst, void const *src,
                                                void *stream) {
    if (desc == nullptr) return STATUS_BAD_DEVICE;
    auto *d = reinterpret_cast<RearrangeDesc *>(desc);
    if (d->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (dst == nullptr || src == nullptr) return STATUS_BAD_PARAM;
    if (d->rows == 0 || d->row_bytes == 0) return STATUS_SUCCESS;
    DeviceGuard guard(d->device_id);
    auto st = reinterpret_cast<cudaStream_t>(stream);
    // the unit also has to divide both base addresses
    int shift = d->gcd_shift;
    const uintptr_t bases = reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src);
    while (shift > 0 && (bases & ((1ull << shift) - 1)) != 0) --shift;
    switch (shift) {
        case 4: return launch<16>(d, dst, src, st);
        case 3: return launch<8>(d, dst, src, st);
        case 2: return launch<4>(d, dst, src, st);
        case 1: return launch<2>(d, dst, src, st);
        default: return launch<1>(d, dst, src, st);
    }
}

INFINIOP_API infiniopStatus_t infiniopDestroyRearrangeDescriptor(infiniopRearrangeDescriptor_t desc) {
    if (desc == nullptr) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<RearrangeDesc *>(desc);
    return STATUS_SUCCESS;
}
