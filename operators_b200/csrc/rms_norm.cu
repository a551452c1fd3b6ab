// RMSNorm: y[n,d] = x[n,d] * rsqrt(mean(x^2) + eps) * w[d], fp16 data, fp16 or
// fp32 weight.
//
// Replaces reference src/ops/rms_norm/cuda/rms_norm.cu:8-173 and
// src/ops/rms_norm/cuda/rms_norm.cc:5-41 behind include/ops/rms_norm/rms_norm.h.
// Arithmetic follows the CPU backend (src/ops/rms_norm/cpu/rms_norm_cpu.cc:
// 63-85): fp32 sum of squares, the scale k = (ss/d + eps)^-1/2 and the product
// k * x * w evaluated in DOUBLE, one rounding to fp32, then the reference's
// truncating fp32 -> fp16 conversion.  Departures: the order of the fp32 sum
// of squares (tree instead of sequential), and in the register kernel the
// product is formed in two-float arithmetic on the fp32 pipe (see rms_prod).
//
// HBM-bound, 4 bytes per element.  A row lives in registers between the
// reduction and the scaling pass, so x is read from HBM exactly once: each
// thread holds up to 8 x 128-bit vectors, a row is owned either by one warp
// (shuffle reduction only) or by one CTA (shuffles + one shared-memory step).
// Rows longer than 32 Ki elements are spread over a thread-block cluster of 2, 4
// or 8 CTAs whose partial sums meet over distributed shared memory (rows of up
// to 256 Ki elements).  Rows that are not 16-byte aligned, or longer still,
// take the two-pass scalar kernel.
//
// The same kernels serve the fused residual form (infiniopAddRMSNorm, which the
// reference does not have): x = a + b with the Add operator's arithmetic
// (src/ops/add/cpu/add_cpu.cc:82-83: exact fp32 sum, truncated to fp16) is
// formed in registers, written out once as the new residual and normalised
// without being read back: 8 bytes per element instead of the 10 of Add
// followed by RMSNorm.
#include "common.cuh"
#include "row_ring.cuh"

#include <new>

using namespace b200;

namespace {

// Many rows of 32768 .. 65536 elements go through the shared-memory ring (measured at 256 MB of rows: 125 against
// 144 us at 32768 elements, 166 against 195 us at 65536; shorter rows are faster from registers, longer ones on the
// register kernels spread over a cluster).
constexpr uint32_t kRingMinVecs = 4096, kRingMaxVecs = 8192;

struct RMSNormDesc {
    Device device;
    int device_id;
    int sm_count;
    uint64_t n, d;
    int64_t stride_y, stride_x;
    bool w_f16;
    float epsilon;
    bool fused;                 // x = a + b, written to `sum`
    int64_t stride_b, stride_sum;
    int dt;                     // kF16, or kBF16 (an extension: bf16 rows and, when 16-bit, weights; same arithmetic)
};

// Second operand and destination of the sum in the fused form.
struct Residual {
    const uint16_t *b;
    uint16_t *sum;
    int64_t stride_b, stride_sum;
};

template<int DT>
__device__ __forceinline__ uint4 add_vec_f16(uint4 x, uint4 y) {
    uint4 r;
    const uint32_t *px = reinterpret_cast<const uint32_t *>(&x);
    const uint32_t *py = reinterpret_cast<const uint32_t *>(&y);
    uint32_t *pr = reinterpret_cast<uint32_t *>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 fx = unpack2_t<DT>(px[k]), fy = unpack2_t<DT>(py[k]);
        pr[k] = pack2_t<DT>(__fadd_rn(fx.x, fy.x), __fadd_rn(fx.y, fy.y));
    }
    return r;
}

__device__ __forceinline__ double h2d(uint16_t h) {
    double r;
    asm("cvt.f64.f16 %0, %1;" : "=d"(r) : "h"(h));
    return r;
}

// (ss / d + eps) ^ -1/2 in double, from the fp32 sum of squares.
__device__ __forceinline__ double rms_scale(float ss, uint64_t d, float eps) {
    const float m = __fadd_rn(__fdiv_rn(ss, (float) d), eps);
    return rsqrt((double) m);
}

template<int DT>
__device__ __forceinline__ double h2d_t(uint16_t h) {
    return DT == kBF16 ? (double) load16<kBF16>(h) : h2d(h);
}
template<int DT>
__device__ __forceinline__ uint16_t rms_out(double k, uint16_t x, double w) {
    return store16<DT>(__double2float_rn(__dmul_rn(__dmul_rn(k, h2d_t<DT>(x)), w)));
}

// The same product on the fp32 pipe (double conversions and multiplies run at a fraction of the fp32 rate
// and would bound the kernel on long inputs): k = k_hi + k_lo as two floats, x * w = p + pe with pe the
// exact residual of the fp32 product (zero for an fp16 weight: 11 + 11 significant bits), and
//   k * x * w = k_hi * p + (k_hi * pe + k_lo * p) + O(2^-48)
// summed smallest first and rounded to fp32 once.  It differs from the double product rounded to fp32
// only when that product lies within 2^-46 (relative) of an fp32 rounding boundary.
struct ScaleF2 {
    float hi, lo;
};
__device__ __forceinline__ ScaleF2 split_scale(double k) {
    ScaleF2 s;
    s.hi = __double2float_rn(k);
    s.lo = __double2float_rn(k - (double) s.hi);
    return s;
}
template<bool W_F16>
__device__ __forceinline__ float rms_prod(ScaleF2 k, float x, float w) {
    const float p = __fmul_rn(x, w);
    const float t = __fmul_rn(k.hi, p);
    float c = __fmaf_rn(k.hi, p, -t);// exact residual of k_hi * p
    c = __fmaf_rn(k.lo, p, c);
    if (!W_F16) c = __fmaf_rn(k.hi, __fmaf_rn(x, w, -p), c);
    return __fadd_rn(t, c);
}

// Who owns a row: one warp (shuffles only), one CTA (shuffles + one shared-memory step) or one thread-block
// cluster (the CTAs' partial sums meet over distributed shared memory).
enum RowOwner { WARP_ROW = 0, CTA_ROW = 1, CLUSTER_ROW = 2 };

// VPT vectors (8 halves each) per thread.  The body is shared by two kernels: one without a launch bound (up to
// 512 threads: the compiler's own register choice, measured faster than any bound) and one bounded to 1024
// threads = 64 registers per thread for the forms that are launched with more than 512.
template<int VPT, bool W_F16, int OWNER, bool FUSED, int DT>
__device__ __forceinline__ void rms_norm_regs_body(uint16_t *y, const uint16_t *x, const void *w, uint64_t n, uint32_t vecs,
                                                   uint64_t d, int64_t stride_y, int64_t stride_x, float eps, Residual res) {
    __shared__ float red[32];
    __shared__ float part;// this CTA's partial sum, read by the whole cluster
    const int lane = threadIdx.x & 31;
    const uint32_t cl = OWNER == CLUSTER_ROW ? cluster_size() : 1;
    const uint32_t group = OWNER == WARP_ROW ? 32 : blockDim.x * cl;
    const uint32_t t = OWNER == WARP_ROW ? lane : (OWNER == CLUSTER_ROW ? cluster_rank() * blockDim.x : 0) + threadIdx.x;
    const uint64_t rows_per_cta = OWNER == WARP_ROW ? (blockDim.x >> 5) : 1;
    const uint64_t row0 = OWNER == WARP_ROW ? (uint64_t) blockIdx.x * rows_per_cta + (threadIdx.x >> 5)
                                            : (uint64_t) (blockIdx.x / cl);
    const uint64_t row_step = OWNER == WARP_ROW ? (uint64_t) gridDim.x * rows_per_cta : (uint64_t) (gridDim.x / cl);

    // CTA / cluster rows: every thread of the CTA (cluster) sees the same row, so the
    // reduction below is reached uniformly; warp rows only use shuffles.
    for (uint64_t row = row0; row < n; row += row_step) {
        const uint16_t *xr = x + (int64_t) row * stride_x;
        uint4 v[VPT];
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            if (j < vecs) v[u] = ld_stream(xr + (uint64_t) j * 8);
        }
        if (FUSED) {
            const uint16_t *br = res.b + (int64_t) row * res.stride_b;
            uint16_t *sr = res.sum + (int64_t) row * res.stride_sum;
            uint4 o[VPT];
#pragma unroll
            for (int u = 0; u < VPT; ++u) {
                const uint32_t j = t + u * group;
                if (j < vecs) o[u] = ld_stream(br + (uint64_t) j * 8);
            }
#pragma unroll
            for (int u = 0; u < VPT; ++u) {
                const uint32_t j = t + u * group;
                if (j < vecs) {
                    v[u] = add_vec_f16<DT>(v[u], o[u]);
                    st_stream(sr + (uint64_t) j * 8, v[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            if (j < vecs) {
                const uint32_t *p = reinterpret_cast<const uint32_t *>(&v[u]);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = unpack2_t<DT>(p[k]);
                    ss = fmaf(f.x, f.x, ss);
                    ss = fmaf(f.y, f.y, ss);
                }
            }
        }
        if (OWNER == CLUSTER_ROW) ss = cluster_reduce<false>(ss, red, &part, cl);
        else ss = OWNER == CTA_ROW ? cta_reduce<false>(ss, red) : warp_sum(ss);
        const ScaleF2 k = split_scale(rms_scale(ss, d, eps));
        uint16_t *yr = y + (int64_t) row * stride_y;
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const uint32_t j = t + u * group;
            if (j < vecs) {
                const uint32_t *px = reinterpret_cast<const uint32_t *>(&v[u]);
                uint4 out;
                uint32_t *po = reinterpret_cast<uint32_t *>(&out);
                if (W_F16) {
                    const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(w) + j);
                    const uint32_t *pw = reinterpret_cast<const uint32_t *>(&wv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 xf = unpack2_t<DT>(px[e]), wf = unpack2_t<DT>(pw[e]);
                        po[e] = pack2_t<DT>(rms_prod<true>(k, xf.x, wf.x), rms_prod<true>(k, xf.y, wf.y));
                    }
                } else {
                    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * j);
                    const float4 w1 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * j + 1);
                    const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 xf = unpack2_t<DT>(px[e]);
                        po[e] = pack2_t<DT>(rms_prod<false>(k, xf.x, wf[2 * e]), rms_prod<false>(k, xf.y, wf[2 * e + 1]));
                    }
                }
                st_stream(yr + (uint64_t) j * 8, out);
            }
        }
        // no CTA may leave (or overwrite `part` for its next row) while a neighbour still reads it
        if (OWNER == CLUSTER_ROW) cluster_sync_all();
    }
}

template<int VPT, bool W_F16, int OWNER, bool FUSED, int MAXT, int DT>
__global__ void rms_norm_regs_kernel(uint16_t *y, const uint16_t *x, const void *w, uint64_t n, uint32_t vecs, uint64_t d,
                                     int64_t stride_y, int64_t stride_x, float eps, Residual res) {
    static_assert(MAXT <= 512, "launches of more than 512 threads use rms_norm_regs_kernel_1024");
    rms_norm_regs_body<VPT, W_F16, OWNER, FUSED, DT>(y, x, w, n, vecs, d, stride_y, stride_x, eps, res);
}
template<int VPT, bool W_F16, int OWNER, bool FUSED, int DT>
__global__ void __launch_bounds__(1024)
    rms_norm_regs_kernel_1024(uint16_t *y, const uint16_t *x, const void *w, uint64_t n, uint32_t vecs, uint64_t d,
                              int64_t stride_y, int64_t stride_x, float eps, Residual res) {
    rms_norm_regs_body<VPT, W_F16, OWNER, FUSED, DT>(y, x, w, n, vecs, d, stride_y, stride_x, eps, res);
}

// Rows of 16 Ki elements and more, many of them: the shared-memory ring of row_ring.cuh (plain form only).
template<bool W_F16, int DT>
__global__ void __launch_bounds__(ring::kThreads, 1)
    rms_norm_ring_kernel(uint16_t *y, const uint16_t *x, const void *w, uint64_t n, uint32_t vecs, uint64_t d,
                         int64_t stride_y, int64_t stride_x, float eps, ring::Plan plan) {
    ring::rms_norm_ring_body<DT, W_F16>(
        y, x, w, n, vecs, d, stride_y, stride_x, eps, plan,
        [](float ss, uint64_t dd, float e) { return split_scale(rms_scale(ss, dd, e)); },
        [](ScaleF2 k, uint4 q, const void *wp, uint32_t j) {
            const uint32_t *px = reinterpret_cast<const uint32_t *>(&q);
            uint4 out;
            uint32_t *po = reinterpret_cast<uint32_t *>(&out);
            if (W_F16) {
                const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(wp) + j);
                const uint32_t *pw = reinterpret_cast<const uint32_t *>(&wv);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 xf = unpack2_t<DT>(px[e]), wf = unpack2_t<DT>(pw[e]);
                    po[e] = pack2_t<DT>(rms_prod<true>(k, xf.x, wf.x), rms_prod<true>(k, xf.y, wf.y));
                }
            } else {
                const float4 w0 = __ldg(reinterpret_cast<const float4 *>(wp) + 2 * j);
                const float4 w1 = __ldg(reinterpret_cast<const float4 *>(wp) + 2 * j + 1);
                const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 xf = unpack2_t<DT>(px[e]);
                    po[e] = pack2_t<DT>(rms_prod<false>(k, xf.x, wf[2 * e]), rms_prod<false>(k, xf.y, wf[2 * e + 1]));
                }
            }
            return out;
        });
}

template<bool W_F16, int DT>
bool launch_ring(const RMSNormDesc *d, uint32_t vecs, void *y, const void *x, const void *w, cudaStream_t st) {
    ring::Plan plan;
    if (!ring::make_plan(plan, vecs, d->n, d->sm_count)) return false;
    auto *kernel = rms_norm_ring_kernel<W_F16, DT>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) plan.smem_bytes) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    auto *yp = reinterpret_cast<uint16_t *>(y);
    auto *xp = reinterpret_cast<const uint16_t *>(x);
    if (plan.cl > 1) {
        launch_cluster_smem(kernel, plan.grid, ring::kThreads, plan.cl, plan.smem_bytes, st, yp, xp, w, d->n, vecs, d->d,
                            d->stride_y, d->stride_x, d->epsilon, plan);
    } else {
        kernel<<<plan.grid, ring::kThreads, plan.smem_bytes, st>>>(yp, xp, w, d->n, vecs, d->d, d->stride_y, d->stride_x,
                                                                  d->epsilon, plan);
    }
    return true;
}

// Any alignment, any d: one CTA per row, two passes over x (the second one is
// served by L2).
template<bool W_F16, bool FUSED, int DT>
__global__ void rms_norm_generic_kernel(uint16_t *y, const uint16_t *x, const void *w, uint64_t n, uint64_t d,
                                        int64_t stride_y, int64_t stride_x, float eps, Residual res) {
    __shared__ float red[32];
    for (uint64_t row = blockIdx.x; row < n; row += gridDim.x) {
        const uint16_t *xr = x + (int64_t) row * stride_x;
        uint16_t *yr = y + (int64_t) row * stride_y;
        float ss = 0.f;
        if (FUSED) {// the sum is written here and read back below by the thread that wrote it
            const uint16_t *br = res.b + (int64_t) row * res.stride_b;
            uint16_t *sr = res.sum + (int64_t) row * res.stride_sum;
            for (uint64_t j = threadIdx.x; j < d; j += blockDim.x) {
                const uint16_t h = store16<DT>(__fadd_rn(load16<DT>(xr[j]), load16<DT>(br[j])));
                sr[j] = h;
                const float f = load16<DT>(h);
                ss = fmaf(f, f, ss);
            }
            xr = sr;
        } else {
            for (uint64_t j = threadIdx.x; j < d; j += blockDim.x) {
                const float f = load16<DT>(xr[j]);
                ss = fmaf(f, f, ss);
            }
        }
        ss = cta_reduce<false>(ss, red);
        const double k = rms_scale(ss, d, eps);
        for (uint64_t j = threadIdx.x; j < d; j += blockDim.x) {
            const double wv = W_F16 ? h2d_t<DT>(reinterpret_cast<const uint16_t *>(w)[j])
                                    : (double) reinterpret_cast<const float *>(w)[j];
            yr[j] = rms_out<DT>(k, xr[j], wv);
        }
        __syncthreads();
    }
}

// false: no register-resident kernel fits this shape (the caller takes the two-pass kernel)
template<int VPT, bool W_F16, bool FUSED, int DT>
bool launch_regs(const RMSNormDesc *d, bool cta_row, uint32_t threads, uint32_t cl, uint32_t vecs, void *y,
                 const void *x, const void *w, Residual res, cudaStream_t st) {
    auto *yp = reinterpret_cast<uint16_t *>(y);
    auto *xp = reinterpret_cast<const uint16_t *>(x);
    if (cta_row) {
        const uint64_t cap = 0x7FFFFFFFull / cl;// one CTA (cluster) per row; rows beyond that loop
        const uint32_t grid = (uint32_t) (d->n < cap ? d->n : cap) * cl;
        if (cl > 1) {
            if constexpr (VPT == 4) {// clusters always hold four vectors per thread
                launch_cluster(rms_norm_regs_kernel_1024<4, W_F16, CLUSTER_ROW, FUSED, DT>, grid, threads, cl, st, yp, xp, w,
                               d->n, vecs, d->d, d->stride_y, d->stride_x, d->epsilon, res);
                return true;
            }
            return false;
        }
        if (threads <= 512 && fits_register_file<rms_norm_regs_kernel<VPT, W_F16, CTA_ROW, FUSED, 512, DT>>(threads)) {
            rms_norm_regs_kernel<VPT, W_F16, CTA_ROW, FUSED, 512, DT>
                <<<grid, threads, 0, st>>>(yp, xp, w, d->n, vecs, d->d, d->stride_y, d->stride_x, d->epsilon, res);
            return true;
        }
        if constexpr (VPT <= 4) {// bounded to 64 registers: any block size
            rms_norm_regs_kernel_1024<VPT, W_F16, CTA_ROW, FUSED, DT>
                <<<grid, threads, 0, st>>>(yp, xp, w, d->n, vecs, d->d, d->stride_y, d->stride_x, d->epsilon, res);
            return true;
        }
        return false;
    }
    const uint64_t ctas = (d->n + 7) / 8;
    const uint64_t cap = 0x7FFFFFFFull;
    const uint32_t grid = (uint32_t) (ctas < cap ? ctas : cap);
    if (!fits_register_file<rms_norm_regs_kernel<VPT, W_F16, WARP_ROW, FUSED, 256, DT>>(256)) return false;
    rms_norm_regs_kernel<VPT, W_F16, WARP_ROW, FUSED, 256, DT>
        <<<grid, 256, 0, st>>>(yp, xp, w, d->n, vecs, d->d, d->stride_y, d->stride_x, d->epsilon, res);
    return true;
}

template<bool W_F16, bool FUSED, int DT>
bool dispatch_regs(const RMSNormDesc *d, int vpt, bool cta_row, uint32_t threads, uint32_t cl, uint32_t vecs, void *y,
                   const void *x, const void *w, Residual res, cudaStream_t st) {
    switch (vpt) {
        case 1: return launch_regs<1, W_F16, FUSED, DT>(d, cta_row, threads, cl, vecs, y, x, w, res, st);
        case 2: return launch_regs<2, W_F16, FUSED, DT>(d, cta_row, threads, cl, vecs, y, x, w, res, st);
        case 4: return launch_regs<4, W_F16, FUSED, DT>(d, cta_row, threads, cl, vecs, y, x, w, res, st);
        default: return launch_regs<8, W_F16, FUSED, DT>(d, cta_row, threads, cl, vecs, y, x, w, res, st);
    }
}

// Kernel choice and launch for both forms; `b` and `sum` are null for the plain one.
template<bool FUSED>
infiniopStatus_t run(const RMSNormDesc *d, void *y, const void *x, const void *w, const void *b, void *sum,
                     cudaStream_t st) {
    const Residual res{reinterpret_cast<const uint16_t *>(b), reinterpret_cast<uint16_t *>(sum), d->stride_b,
                       d->stride_sum};
    // rows of up to 8 CTAs x 1024 threads x 4 vectors stay in registers; longer ones go the scalar way
    bool vec_ok = d->d % 8 == 0 && d->d / 8 <= 32768 && d->stride_x % 8 == 0 && d->stride_y % 8 == 0 &&
                  aligned16(y) && aligned16(x) && aligned16(w);
    if (FUSED) {
        vec_ok = vec_ok && d->stride_b % 8 == 0 && d->stride_sum % 8 == 0 && aligned16(b) && aligned16(sum);
    }
    if (vec_ok) {
        const uint32_t vecs = (uint32_t) (d->d / 8);
        // Enough rows to fill the GPU: favour bytes in flight per thread (8
        // vectors each, a warp per row when the row fits).  Few rows: favour
        // latency, spread each row over as many threads as it has vectors.
        const bool big = d->n * (uint64_t) vecs >= (1u << 20);
        // infiniopExtSelectKernel(long rows, 1) keeps the register kernels, 2 takes the ring for every row of 4096
        // elements and more
        const int ring_choice = kernel_choice(kFamilyLongRows);
        if (!FUSED && ring_choice != 1 && ((big && vecs >= kRingMinVecs && vecs <= kRingMaxVecs) || (ring_choice == 2 && vecs >= 512))) {
            const bool launched = d->dt == kBF16 ? (d->w_f16 ? launch_ring<true, kBF16>(d, vecs, y, x, w, st)
                                                            : launch_ring<false, kBF16>(d, vecs, y, x, w, st))
                                                 : (d->w_f16 ? launch_ring<true, kF16>(d, vecs, y, x, w, st)
                                                            : launch_ring<false, kF16>(d, vecs, y, x, w, st));
            if (launched) return check_launch("rms_norm (ring)");
        }
        int vpt;
        bool cta_row;
        uint32_t threads = 256, cl = 1;
        if (big && vecs <= (FUSED ? 128u : 256u)) {// the fused form holds two operands: half the vectors per thread
            cta_row = false;
            const uint32_t need = (vecs + 31) / 32;
            vpt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
        } else {
            cta_row = true;
            // measured on [32768, 4096] / [16384, 8192] / [8192, 16384] with one CTA per row: 4 vectors per thread
            // 0.88 / 0.87 / 0.81 of the copy bandwidth, 8 vectors 0.79 / 0.78 / 0.70, 2 vectors 0.75 / 0.71 / 0.59.
            // Rows of more than 4096 vectors are spread over a cluster of 2, 4 or 8 CTAs.
            const RowLaunch shape = row_launch_shape(vecs, big ? (FUSED ? 2 : 4) : 1);
            vpt = shape.vpt, threads = shape.threads, cl = shape.cl;
        }
        bool launched;
        if (d->dt == kBF16) {
            launched = d->w_f16 ? dispatch_regs<true, FUSED, kBF16>(d, vpt, cta_row, threads, cl, vecs, y, x, w, res, st)
                                : dispatch_regs<false, FUSED, kBF16>(d, vpt, cta_row, threads, cl, vecs, y, x, w, res, st);
        } else {
            launched = d->w_f16 ? dispatch_regs<true, FUSED, kF16>(d, vpt, cta_row, threads, cl, vecs, y, x, w, res, st)
                                : dispatch_regs<false, FUSED, kF16>(d, vpt, cta_row, threads, cl, vecs, y, x, w, res, st);
        }
        if (launched) return check_launch("rms_norm");
    }
    const uint64_t cap = (uint64_t) d->sm_count * 8;
    const uint32_t grid = (uint32_t) (d->n < cap ? d->n : cap);
    auto *yp = reinterpret_cast<uint16_t *>(y);
    auto *xp = reinterpret_cast<const uint16_t *>(x);
    auto *generic = d->dt == kBF16 ? (d->w_f16 ? rms_norm_generic_kernel<true, FUSED, kBF16> : rms_norm_generic_kernel<false, FUSED, kBF16>)
                                   : (d->w_f16 ? rms_norm_generic_kernel<true, FUSED, kF16> : rms_norm_generic_kernel<false, FUSED, kF16>);
    generic<<<grid, 256, 0, st>>>(yp, xp, w, d->n, d->d, d->stride_y, d->stride_x, d->epsilon, res);
    return check_launch("rms_norm");
}

}// namespace

namespace b200 {
unsigned long long rms_norm_ring_timeouts_read() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, ring::g_row_ring_timeouts, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return ~0ull;
    }
    return v;
}
}// namespace b200

INFINIOP_API infiniopStatus_t infiniopCreateRMSNormDescriptor(infiniopHandle_t handle,
                                                              infiniopRMSNormDescriptor_t *desc_ptr,
                                                              infiniopTensorDescriptor_t y_desc,
                                                              infiniopTensorDescriptor_t x_desc,
                                                              infiniopTensorDescriptor_t w_desc, float epsilon) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (y_desc == nullptr || x_desc == nullptr || w_desc == nullptr) return STATUS_BAD_PARAM;
    // Shape checks and codes of reference rms_norm.cc:10-19.
    if (y_desc->ndim != 2 || x_desc->ndim != 2 || w_desc->ndim != 1) return STATUS_BAD_TENSOR_SHAPE;
    const uint64_t n = y_desc->shape[0], d = y_desc->shape[1];
    if (x_desc->shape[0] != n || x_desc->shape[1] != d || w_desc->shape[0] != d) return STATUS_BAD_TENSOR_SHAPE;
    // The reference defers the dtype check to the compute call
    // (rms_norm.cu:165-171: anything but fp16 data -> BAD_TENSOR_DTYPE) and reads
    // any non-fp16 weight as fp32; the weight must really be one of the two here.
    // bf16 rows are an extension of this library: x and y bf16, the weight bf16 or fp32
    const int dt = store_type_of(y_desc->dt);
    if ((dt != kF16 && dt != kBF16) || !dt_eq(x_desc->dt, y_desc->dt)) return STATUS_BAD_TENSOR_DTYPE;
    if (!dt_eq(w_desc->dt, y_desc->dt) && !dt_eq(w_desc->dt, F32)) return STATUS_BAD_TENSOR_DTYPE;
    if (y_desc->strides[1] != 1 || x_desc->strides[1] != 1 || w_desc->strides[0] != 1) return STATUS_BAD_TENSOR_STRIDES;

    auto *h = reinterpret_cast<Handle *>(handle);
    auto *r = new (std::nothrow) RMSNormDesc{DevNvGpu, h->device_id,         h->sm_count,           n,
                                             d,        y_desc->strides[0],   x_desc->strides[0],    !dt_eq(w_desc->dt, F32),
                                             epsilon,  false,                0,                     0,
                                             dt};
    if (r == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    *desc_ptr = reinterpret_cast<infiniopRMSNormDescriptor_t>(r);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetRMSNormWorkspaceSize(infiniopRMSNormDescriptor_t desc, uint64_t *size) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = 0;
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopRMSNorm(infiniopRMSNormDescriptor_t desc, void *workspace,
                                              uint64_t workspace_size, void *y, void const *x, void const *w,
                                              void *stream) {
    (void) workspace;
    (void) workspace_size;
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (y == nullptr || x == nullptr || w == nullptr) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<RMSNormDesc *>(desc);
    if (d->fused) return STATUS_BAD_PARAM;// a descriptor of the fused form
    if (d->n == 0 || d->d == 0) return STATUS_SUCCESS;
    DeviceGuard guard(d->device_id);
    auto st = reinterpret_cast<cudaStream_t>(stream);
    return run<false>(d, y, x, w, nullptr, nullptr, st);
}

INFINIOP_API infiniopStatus_t infiniopDestroyRMSNormDescriptor(infiniopRMSNormDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<RMSNormDesc *>(desc);
    return STATUS_SUCCESS;
}

// ---- fused residual form: sum = a + b, y = RMSNorm(sum) * w (no counterpart in the reference) ----------------
INFINIOP_API infiniopStatus_t infiniopCreateAddRMSNormDescriptor(infiniopHandle_t handle,
                                                                 infiniopAddRMSNormDescriptor_t *desc_ptr,
                                                                 infiniopTensorDescriptor_t y_desc,
                                                                 infiniopTensorDescriptor_t sum_desc,
                                                                 infiniopTensorDescriptor_t a_desc,
                                                                 infiniopTensorDescriptor_t b_desc,
                                                                 infiniopTensorDescriptor_t w_desc, float epsilon) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (y_desc == nullptr || sum_desc == nullptr || a_desc == nullptr || b_desc == nullptr || w_desc == nullptr) {
        return STATUS_BAD_PARAM;
    }
    // the checks of the RMSNorm descriptor, applied to all four row tensors; no broadcasting
    infiniopTensorDescriptor_t rows[4] = {y_desc, sum_desc, a_desc, b_desc};
    for (auto *t : rows) {
        if (t->ndim != 2) return STATUS_BAD_TENSOR_SHAPE;
    }
    if (w_desc->ndim != 1) return STATUS_BAD_TENSOR_SHAPE;
    const uint64_t n = y_desc->shape[0], d = y_desc->shape[1];
    for (auto *t : rows) {
        if (t->shape[0] != n || t->shape[1] != d) return STATUS_BAD_TENSOR_SHAPE;
    }
    if (w_desc->shape[0] != d) return STATUS_BAD_TENSOR_SHAPE;
    const int dt = store_type_of(y_desc->dt);
    if (dt != kF16 && dt != kBF16) return STATUS_BAD_TENSOR_DTYPE;
    for (auto *t : rows) {
        if (!dt_eq(t->dt, y_desc->dt)) return STATUS_BAD_TENSOR_DTYPE;
    }
    if (!dt_eq(w_desc->dt, y_desc->dt) && !dt_eq(w_desc->dt, F32)) return STATUS_BAD_TENSOR_DTYPE;
    for (auto *t : rows) {
        if (t->strides[1] != 1) return STATUS_BAD_TENSOR_STRIDES;
    }
    if (w_desc->strides[0] != 1) return STATUS_BAD_TENSOR_STRIDES;

    auto *h = reinterpret_cast<Handle *>(handle);
    auto *r = new (std::nothrow) RMSNormDesc{DevNvGpu, h->device_id,        h->sm_count,          n,
                                             d,        y_desc->strides[0],  a_desc->strides[0],   !dt_eq(w_desc->dt, F32),
                                             epsilon,  true,                b_desc->strides[0],   sum_desc->strides[0],
                                             dt};
    if (r == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    *desc_ptr = reinterpret_cast<infiniopAddRMSNormDescriptor_t>(r);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetAddRMSNormWorkspaceSize(infiniopAddRMSNormDescriptor_t desc, uint64_t *size) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = 0;
    return STATUS_SUCCESS;
}

// `sum` may be `a` or `b` (the residual updated in place); `y` must not overlap `sum`.
INFINIOP_API infiniopStatus_t infiniopAddRMSNorm(infiniopAddRMSNormDescriptor_t desc, void *workspace,
                                                 uint64_t workspace_size, void *y, void *sum, void const *a,
                                                 void const *b, void const *w, void *stream) {
    (void) workspace;
    (void) workspace_size;
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (y == nullptr || sum == nullptr || a == nullptr || b == nullptr || w == nullptr) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<RMSNormDesc *>(desc);
    if (!d->fused) return STATUS_BAD_PARAM;
    if (d->n == 0 || d->d == 0) return STATUS_SUCCESS;
    DeviceGuard guard(d->device_id);
    return run<true>(d, y, a, w, b, sum, reinterpret_cast<cudaStream_t>(stream));
}

INFINIOP_API infiniopStatus_t infiniopDestroyAddRMSNormDescriptor(infiniopAddRMSNormDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<RMSNormDesc *>(desc);
    return STATUS_SUCCESS;
}
