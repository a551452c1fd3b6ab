// Add: c = a + b with numpy-style broadcasting, contiguous fp16 / fp32 tensors (and bf16, an extension: see
// StoreType in common.cuh).
//
// Replaces reference src/ops/add/cuda/add.cu:12-116 and src/ops/add/cuda/add.cc:
// 5-73 behind include/ops/add/add.h.  Arithmetic follows the CPU backend
// (src/ops/add/cpu/add_cpu.cc:72-89): fp16 operands are widened, added in fp32
// (round to nearest) and narrowed with the reference's truncating conversion;
// fp32 is a plain add.  Both are reproduced bit for bit.
//
// HBM-bound, 3 streams.  Without broadcasting the three tensors are flat
// arrays: one 256-thread CTA per tile of 1024 vectors, 4 x 128-bit loads per
// thread per stream in flight (one tile per CTA measured faster on B200 than a
// persistent grid-stride loop).  With broadcasting, dimensions are collapsed on
// the host and the per-axis strides travel in the kernel arguments (the
// reference cudaMallocs three stride arrays per descriptor, add.cc:48-54;
// nothing is allocated on the device here).
#include "common.cuh"
#include "fastdiv.h"

#include <new>
#include <type_traits>

using namespace b200;

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kMaxDims = 8;

struct BroadcastDims {
    int ndim;
    uint32_t shape[kMaxDims];// collapsed c shape, outermost first
    int64_t sa[kMaxDims];    // a stride per collapsed axis (0 = broadcast)
    int64_t sb[kMaxDims];
};

struct AddDesc {
    Device device;
    int device_id;
    int sm_count;
    int dt;// StoreType
    bool broadcast;
    uint64_t total;// elements of c
    BroadcastDims dims;
};

template<int DT>
__device__ __forceinline__ uint4 add_vec(uint4 x, uint4 y) {
    constexpr bool F16 = DT != kF32;// 16-bit storage
    uint4 r;
    const uint32_t *px = reinterpret_cast<const uint32_t *>(&x);
    const uint32_t *py = reinterpret_cast<const uint32_t *>(&y);
    uint32_t *pr = reinterpret_cast<uint32_t *>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (F16) {
            float2 fx = unpack2_t<DT>(px[k]), fy = unpack2_t<DT>(py[k]);
            pr[k] = pack2_t<DT>(__fadd_rn(fx.x, fy.x), __fadd_rn(fx.y, fy.y));
        } else {
            pr[k] = __float_as_uint(__fadd_rn(__uint_as_float(px[k]), __uint_as_float(py[k])));
        }
    }
    return r;
}

template<int DT>
__global__ void __launch_bounds__(kThreads)
    add_flat_kernel(void *c, const void *a, const void *b, uint64_t total_vecs, uint64_t total) {
    constexpr bool F16 = DT != kF32;
    const uint4 *av = reinterpret_cast<const uint4 *>(a);
    const uint4 *bv = reinterpret_cast<const uint4 *>(b);
    uint4 *cv = reinterpret_cast<uint4 *>(c);
    {
        const uint64_t base = (uint64_t) blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
        uint4 x[kUnroll], y[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint64_t v = base + (uint64_t) u * kThreads;
            if (v < total_vecs) {
                x[u] = ld_stream(av + v);
                y[u] = ld_stream(bv + v);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint64_t v = base + (uint64_t) u * kThreads;
            if (v < total_vecs) st_stream(cv + v, add_vec<DT>(x[u], y[u]));
        }
    }
    // Fewer than one vector of elements may remain at the end.
    constexpr uint64_t per_vec = F16 ? 8 : 4;
    const uint64_t done = total_vecs * per_vec;
    if (blockIdx.x == 0 && done + threadIdx.x < total) {
        const uint64_t i = done + threadIdx.x;
        if (F16) {
            auto *cp = reinterpret_cast<uint16_t *>(c);
            cp[i] = store16<DT>(__fadd_rn(load16<DT>(reinterpret_cast<const uint16_t *>(a)[i]),
                                          load16<DT>(reinterpret_cast<const uint16_t *>(b)[i])));
        } else {
            reinterpret_cast<float *>(c)[i] =
                __fadd_rn(reinterpret_cast<const float *>(a)[i], reinterpret_cast<const float *>(b)[i]);
        }
    }
}

// Any alignment and any broadcast pattern: one element per thread per step,
// operand offsets rebuilt from the collapsed multi-index.
template<int DT, bool FLAT>
__global__ void __launch_bounds__(kThreads)
    add_general_kernel(void *c, const void *a, const void *b, uint64_t total, BroadcastDims dims) {
    constexpr bool F16 = DT != kF32;
    for (uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x; i < total; i += (uint64_t) gridDim.x * kThreads) {
        uint64_t rem = i;
        int64_t oa = FLAT ? (int64_t) i : 0, ob = oa;
        if (!FLAT) {
#pragma unroll 1
            for (int ax = dims.ndim - 1; ax >= 0; --ax) {
                const uint64_t q = rem / dims.shape[ax];
                const uint64_t idx = rem - q * dims.shape[ax];
                oa += (int64_t) idx * dims.sa[ax];
                ob += (int64_t) idx * dims.sb[ax];
                rem = q;
            }
        }
        if (F16) {
            reinterpret_cast<uint16_t *>(c)[i] =
                store16<DT>(__fadd_rn(load16<DT>(reinterpret_cast<const uint16_t *>(a)[oa]),
                                      load16<DT>(reinterpret_cast<const uint16_t *>(b)[ob])));
        } else {
            reinterpret_cast<float *>(c)[i] =
                __fadd_rn(reinterpret_cast<const float *>(a)[oa], reinterpret_cast<const float *>(b)[ob]);
        }
    }
}

// Broadcast patterns whose innermost collapsed axis is walked with stride 1 or 0 by both operands and
// is a whole number of 128-bit vectors long: one vector of c per thread and step; the vector's multi-index
// is rebuilt once (multiply-high dividers, the innermost extent counted in vectors), an operand that does
// not span the innermost axis contributes one replicated element.  Everything else (odd extents,
// unaligned bases) stays on add_general_kernel.
struct VecDims {
    int ndim;
    FastDiv div[kMaxDims];// extents, the innermost one in vectors
    int64_t sa[kMaxDims]; // strides in elements; for the innermost axis per vector (V or 0)
    int64_t sb[kMaxDims];
    bool a_inner, b_inner;// operand spans the innermost axis
};

template<int DT>
__global__ void __launch_bounds__(kThreads)
    add_bcast_vec_kernel(void *c, const void *a, const void *b, uint32_t total_vecs, VecDims dims) {
    constexpr bool F16 = DT != kF32;
    constexpr int V = F16 ? 8 : 4;
    using E = typename std::conditional<F16, uint16_t, uint32_t>::type;
    const E *ae = reinterpret_cast<const E *>(a), *be = reinterpret_cast<const E *>(b);
    uint4 *cv = reinterpret_cast<uint4 *>(c);
    const uint32_t base = blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
    uint4 x[kUnroll], y[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const uint32_t v = base + u * kThreads;
        if (v < total_vecs) {
            uint32_t rem = v;
            int64_t oa = 0, ob = 0;
            for (int ax = dims.ndim - 1; ax >= 0; --ax) {
                uint32_t q, idx;
                dims.div[ax].divmod(rem, q, idx);
                oa += (int64_t) idx * dims.sa[ax];
                ob += (int64_t) idx * dims.sb[ax];
                rem = q;
            }
            if (dims.a_inner) {
                x[u] = ld_stream(ae + oa);
            } else {
                const uint32_t e = F16 ? (uint32_t) ae[oa] * 0x00010001u : (uint32_t) ae[oa];
                x[u] = make_uint4(e, e, e, e);
            }
            if (dims.b_inner) {
                y[u] = ld_stream(be + ob);
            } else {
                const uint32_t e = F16 ? (uint32_t) be[ob] * 0x00010001u : (uint32_t) be[ob];
                y[u] = make_uint4(e, e, e, e);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const uint32_t v = base + u * kThreads;
        if (v < total_vecs) st_stream(cv + v, add_vec<DT>(x[u], y[u]));
    }
}

// Row-major contiguity over all axes (reference src/ops/utils.h:174-188).  The
// reference only compares neighbouring strides, so a tensor whose innermost
// stride is 2 passes there and is then read as if it were dense; here the
// innermost stride must be 1 as well.
bool contiguous(infiniopTensorDescriptor_t t) {
    if (t->ndim > 0 && t->shape[t->ndim - 1] > 1 && t->strides[t->ndim - 1] != 1) return false;
    for (uint64_t i = 1; i < t->ndim; ++i) {
        if (t->strides[i - 1] != (int64_t) t->shape[i] * t->strides[i]) return false;
    }
    return true;
}

// c.shape must equal broadcast(a.shape, b.shape) and have max(a.ndim, b.ndim)
// axes (reference src/ops/utils.h:85-143).
bool valid_broadcast(infiniopTensorDescriptor_t a, infiniopTensorDescriptor_t b, infiniopTensorDescriptor_t c) {
    const uint64_t nd = a->ndim > b->ndim ? a->ndim : b->ndim;
    if (c->ndim != nd) return false;
    for (uint64_t i = 0; i < nd; ++i) {
        const uint64_t da = i < nd - a->ndim ? 1 : a->shape[i - (nd - a->ndim)];
        const uint64_t db = i < nd - b->ndim ? 1 : b->shape[i - (nd - b->ndim)];
        if (!(da == db || da == 1 || db == 1)) return false;
        const uint64_t out = da > db ? da : db;
        if (out != c->shape[i]) return false;
    }
    return true;
}

}// namespace

INFINIOP_API infiniopStatus_t infiniopCreateAddDescriptor(infiniopHandle_t handle, infiniopAddDescriptor_t *desc_ptr,
                                                          infiniopTensorDescriptor_t c, infiniopTensorDescriptor_t a,
                                                          infiniopTensorDescriptor_t b) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (c == nullptr || a == nullptr || b == nullptr) return STATUS_BAD_PARAM;
    // Same checks, same order, same codes as reference add.cc:11-23.
    if (!valid_broadcast(a, b, c)) return STATUS_BAD_TENSOR_SHAPE;
    if (!contiguous(a) || !contiguous(b) || !contiguous(c)) return STATUS_BAD_TENSOR_STRIDES;
    if (store_type_of(c->dt) < 0) return STATUS_BAD_TENSOR_DTYPE;// fp16, fp32 (reference) or bf16 (extension)
    if (!dt_eq(c->dt, a->dt) || !dt_eq(c->dt, b->dt)) return STATUS_BAD_TENSOR_DTYPE;

    const uint64_t nd = c->ndim;
    bool broadcast = (nd != a->ndim || nd != b->ndim);
    for (uint64_t i = 0; i < nd && !broadcast; ++i) {
        broadcast = c->shape[i] != a->shape[i] || c->shape[i] != b->shape[i];
    }
    uint64_t total = 1;
    for (uint64_t i = 0; i < nd; ++i) total *= c->shape[i];

    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow) AddDesc{};
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    d->device = DevNvGpu;
    d->device_id = h->device_id;
    d->sm_count = h->sm_count;
    d->dt = store_type_of(c->dt);
    d->broadcast = broadcast;
    d->total = total;
    d->dims.ndim = 0;

    if (broadcast) {
        // Adjusted strides (0 on an axis the operand does not span; reference
        // add.cc:40-45), then merge neighbouring axes that both operands walk
        // as one run, and drop axes of extent 1.
        BroadcastDims &bd = d->dims;
        for (uint64_t i = 0; i < nd; ++i) {
            const uint64_t ext = c->shape[i];
            if (ext == 1) continue;
            const bool a_has = i >= nd - a->ndim && a->shape[i - (nd - a->ndim)] == ext;
            const bool b_has = i >= nd - b->ndim && b->shape[i - (nd - b->ndim)] == ext;
            const int64_t sa = a_has ? a->strides[i - (nd - a->ndim)] : 0;
            const int64_t sb = b_has ? b->strides[i - (nd - b->ndim)] : 0;
            if (bd.ndim > 0) {
                const int p = bd.ndim - 1;
                const bool merge = bd.sa[p] == sa * (int64_t) ext && bd.sb[p] == sb * (int64_t) ext &&
                                   (uint64_t) bd.shape[p] * ext <= 0xFFFFFFFFull;
                if (merge) {
                    bd.shape[p] = (uint32_t) (bd.shape[p] * ext);
                    bd.sa[p] = sa;
                    bd.sb[p] = sb;
                    continue;
                }
            }
            if (bd.ndim == kMaxDims || ext > 0xFFFFFFFFull) {
                delete d;
                return STATUS_BAD_TENSOR_SHAPE;// more than 8 non-mergeable axes
            }
            bd.shape[bd.ndim] = (uint32_t) ext;
            bd.sa[bd.ndim] = sa;
            bd.sb[bd.ndim] = sb;
            ++bd.ndim;
        }
    }
    *desc_ptr = reinterpret_cast<infiniopAddDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopAdd(infiniopAddDescriptor_t desc, void *c, void const *a, void const *b,
                                          void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (c == nullptr || a == nullptr || b == nullptr) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<AddDesc *>(desc);
    if (d->total == 0) return STATUS_SUCCESS;
    DeviceGuard guard(d->device_id);
    auto st = reinterpret_cast<cudaStream_t>(stream);

    if (!d->broadcast && aligned16(c) && aligned16(a) && aligned16(b)) {
        const uint64_t per_vec = d->dt != kF32 ? 8 : 4;
        const uint64_t vecs = d->total / per_vec;
        const uint64_t tiles = (vecs + kThreads * kUnroll - 1) / (kThreads * kUnroll);
        if (tiles > 0x7FFFFFFFull) return STATUS_BAD_TENSOR_SHAPE;// > 2^41 elements
        const uint64_t grid = tiles == 0 ? 1 : tiles;
        if (d->dt == kF16) add_flat_kernel<kF16><<<(uint32_t) grid, kThreads, 0, st>>>(c, a, b, vecs, d->total);
        else if (d->dt == kBF16) add_flat_kernel<kBF16><<<(uint32_t) grid, kThreads, 0, st>>>(c, a, b, vecs, d->total);
        else add_flat_kernel<kF32><<<(uint32_t) grid, kThreads, 0, st>>>(c, a, b, vecs, d->total);
        return check_launch("add");
    }
    if (d->broadcast && d->dims.ndim >= 1 && aligned16(c) && aligned16(a) && aligned16(b)) {
        const BroadcastDims &bd = d->dims;
        const int in = bd.ndim - 1;
        const uint32_t V = d->dt != kF32 ? 8u : 4u;
        bool ok = bd.shape[in] % V == 0 && (bd.sa[in] == 0 || bd.sa[in] == 1) && (bd.sb[in] == 0 || bd.sb[in] == 1) &&
                  d->total / V <= 0xFFFFFFFFull;
        VecDims vd;
        vd.ndim = bd.ndim;
        vd.a_inner = bd.sa[in] == 1;
        vd.b_inner = bd.sb[in] == 1;
        for (int ax = 0; ax < bd.ndim && ok; ++ax) {
            const bool inner = ax == in;
            vd.div[ax] = FastDiv(inner ? bd.shape[ax] / V : bd.shape[ax]);
            vd.sa[ax] = inner ? bd.sa[ax] * (int64_t) V : bd.sa[ax];
            vd.sb[ax] = inner ? bd.sb[ax] * (int64_t) V : bd.sb[ax];
            // vector loads of an operand that spans the innermost axis need every outer step to keep 16-byte alignment
            if (!inner && ((vd.a_inner && bd.sa[ax] % V != 0) || (vd.b_inner && bd.sb[ax] % V != 0))) ok = false;
        }
        if (ok) {
            const uint32_t vecs = (uint32_t) (d->total / V);
            const uint32_t tiles = (vecs + kThreads * kUnroll - 1) / (kThreads * kUnroll);
            if (d->dt == kF16) add_bcast_vec_kernel<kF16><<<tiles, kThreads, 0, st>>>(c, a, b, vecs, vd);
            else if (d->dt == kBF16) add_bcast_vec_kernel<kBF16><<<tiles, kThreads, 0, st>>>(c, a, b, vecs, vd);
            else add_bcast_vec_kernel<kF32><<<tiles, kThreads, 0, st>>>(c, a, b, vecs, vd);
            return check_launch("add");
        }
    }
    // Broadcast, or flat tensors at addresses that are not 16-byte aligned.
    uint64_t blocks = (d->total + kThreads - 1) / kThreads;
    const uint64_t cap = (uint64_t) d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    const uint32_t g = (uint32_t) blocks;
    if (d->broadcast) {
        if (d->dt == kF16) add_general_kernel<kF16, false><<<g, kThreads, 0, st>>>(c, a, b, d->total, d->dims);
        else if (d->dt == kBF16) add_general_kernel<kBF16, false><<<g, kThreads, 0, st>>>(c, a, b, d->total, d->dims);
        else add_general_kernel<kF32, false><<<g, kThreads, 0, st>>>(c, a, b, d->total, d->dims);
    } else {
        if (d->dt == kF16) add_general_kernel<kF16, true><<<g, kThreads, 0, st>>>(c, a, b, d->total, d->dims);
        else if (d->dt == kBF16) add_general_kernel<kBF16, true><<<g, kThreads, 0, st>>>(c, a, b, d->total, d->dims);
        else add_general_kernel<kF32, true><<<g, kThreads, 0, st>>>(c, a, b, d->total, d->dims);
    }
    return check_launch("add");
}

INFINIOP_API infiniopStatus_t infiniopDestroyAddDescriptor(infiniopAddDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<AddDesc *>(desc);
    return STATUS_SUCCESS;
}
