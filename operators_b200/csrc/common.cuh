// Shared device/host toolkit of the sm_100a backend: descriptor helpers, the
// reference's fp16 rounding rule, 128-bit streaming accesses, warp / CTA
// reductions and an exact 32-bit divider for flat-index -> (row, column) math.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/infiniop.h"
#include "fastdiv.h"

namespace b200 {

// ---------------------------------------------------------------- host side --

// 32-bit image of a DataLayout; the reference compares layouts the same way
// (reference src/ops/utils.h:62-72).
static inline uint32_t dt_bits(DataLayout d) {
    union {
        DataLayout l;
        uint32_t u;
    } p;
    p.u = 0;
    p.l = d;
    return p.u;
}
static inline bool dt_eq(DataLayout a, DataLayout b) { return dt_bits(a) == dt_bits(b); }

// Handle object behind infiniopHandle_t: first field is the device enum, as the
// reference's CudaContext (reference src/devices/cuda/cuda_handle.h:12-20).
struct Handle {
    Device device;
    int device_id;
    int sm_count;
    int max_smem_optin;
};

// RAII "run on this device" guard used by every compute entry point: the
// reference calls cudaSetDevice(desc->device_id) in most of them
// (e.g. reference src/ops/rms_norm/cuda/rms_norm.cu:164) and never restores it;
// restoring keeps multi-GPU hosts (one handle per GPU in one thread) sane.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) {
            switched = cudaSetDevice(dev) == cudaSuccess;
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

// Launch errors are reported like the reference reports CUDA API failures
// (reference src/devices/cuda/common_cuda.h:10-32): a line on stderr and a
// status code; nothing throws across the C ABI.
static inline infiniopStatus_t check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "infiniop[b200]: %s launch failed: %s\n", what, cudaGetErrorString(e));
        return STATUS_EXECUTION_FAILED;
    }
    return STATUS_SUCCESS;
}

// Kernel-family override set through infiniopExtSelectKernel (runtime.cu); 0 = the library's own choice.
enum KernelFamily { kFamilyRoPE = 0, kFamilyRandomSample = 1, kFamilyAttention = 2, kFamilyMatmul = 3, kFamilyLongRows = 4, kFamilyCount = 8 };
int kernel_choice(int family);

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline bool aligned4(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

// -------------------------------------------------------------- device side --

// fp32 -> fp16 with the reference CPU backend's rule (reference
// src/devices/cpu/common_cpu.cc:41-64): mantissa TRUNCATED, |x| < 2^-24 to
// signed zero, NaN -> sign|0x7E00, and for finite |x| >= 65536 the raw
// `sign | ((e+15) << 10) | (mantissa >> 13)` with the exponent field spilling
// into bit 15.  cvt.rz agrees with that rule everywhere below 65536, so the
// integer path is only taken for the out-of-range tail and NaN.
__device__ __forceinline__ uint16_t f32_to_f16_ref(float v) {
    uint32_t u = __float_as_uint(v);
    uint32_t au = u & 0x7FFFFFFFu;
    if (au < 0x47800000u) {// |v| < 65536
        return __half_as_ushort(__float2half_rz(v));
    }
    uint32_t sign = (u >> 16) & 0x8000u;
    int32_t e = (int32_t) ((u >> 23) & 0xFFu) - 127;
    uint32_t man = u & 0x7FFFFFu;
    if (e >= 31) {
        return (uint16_t) ((e == 128 && man != 0) ? (sign | 0x7E00u) : (sign | 0x7C00u));
    }
    return (uint16_t) (sign | ((uint32_t) (e + 15) << 10) | (man >> 13));
}

__device__ __forceinline__ float f16_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// Two conversions at once: one packed cvt.rz when both values are in range,
// the element-wise rule otherwise.
__device__ __forceinline__ uint32_t pack2_ref(float lo, float hi) {
    if (fmaxf(fabsf(lo), fabsf(hi)) < 65536.0f) {// false for NaN as well
        uint32_t r;
        asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    return (uint32_t) f32_to_f16_ref(lo) | ((uint32_t) f32_to_f16_ref(hi) << 16);
}
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&w));
}

// ---- storage types -------------------------------------------------------------------------------------
// fp16 is the reference's type.  bf16 storage is an extension of this library (the reference only carries the
// BF16 layout constant, include/data_type.h:44): the same arithmetic in fp32 with bf16 decode (exact: the upper
// half of the fp32 pattern) and encode by TRUNCATION of the mantissa, the counterpart of the reference's
// truncating fp16 rule; NaN stays NaN (sign | 0x7FC0).
enum StoreType { kF32 = 0, kF16 = 1, kBF16 = 2 };

static inline int store_type_of(DataLayout d) { return dt_eq(d, F16) ? kF16 : dt_eq(d, BF16) ? kBF16 : dt_eq(d, F32) ? kF32 : -1; }

__device__ __forceinline__ uint16_t f32_to_bf16_trunc(float v) {
    const uint32_t u = __float_as_uint(v);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t) (((u >> 16) & 0x8000u) | 0x7FC0u);
    return (uint16_t) (u >> 16);
}
template<int DT>
__device__ __forceinline__ float load16(uint16_t h) {
    return DT == kBF16 ? __uint_as_float((uint32_t) h << 16) : f16_to_f32(h);
}
template<int DT>
__device__ __forceinline__ uint16_t store16(float v) {
    return DT == kBF16 ? f32_to_bf16_trunc(v) : f32_to_f16_ref(v);
}
// two elements per 32-bit word
template<int DT>
__device__ __forceinline__ float2 unpack2_t(uint32_t w) {
    if (DT == kBF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    return unpack2(w);
}
template<int DT>
__device__ __forceinline__ uint32_t pack2_t(float lo, float hi) {
    if (DT == kBF16) return (uint32_t) f32_to_bf16_trunc(lo) | ((uint32_t) f32_to_bf16_trunc(hi) << 16);
    return pack2_ref(lo, hi);
}

// 2^x by the special-function unit (ex2.approx: relative error about 2^-22,
// -inf -> +0, results below 2^-126 flush to zero).
__device__ __forceinline__ float fast_exp2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
constexpr float kLog2e = 1.4426950408889634f;

// 128-bit accesses with the streaming (evict-first) policy.  Loads are
// ordinary coherent loads, not the read-only path, so operators whose output
// aliases an input (in-place SwiGLU / Add / RoPE / softmax) stay well defined.
__device__ __forceinline__ uint4 ld_stream(const void *p) { return __ldcs(reinterpret_cast<const uint4 *>(p)); }
__device__ __forceinline__ void st_stream(void *p, uint4 v) { __stcs(reinterpret_cast<uint4 *>(p), v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// CTA-wide reduction for kernels that give one whole CTA to a row.  `slot` is
// 32 floats of shared memory; all threads of the CTA must call it.
template<bool IS_MAX>
__device__ __forceinline__ float cta_reduce(float v, float *slot) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    if (nwarps == 1) return v;
    if (lane == 0) slot[warp] = v;
    __syncthreads();
    float r = slot[0];
    for (int w = 1; w < nwarps; ++w) r = IS_MAX ? fmaxf(r, slot[w]) : r + slot[w];
    __syncthreads();
    return r;
}

// The same with a single barrier: the caller alternates between two slots (e.g. one for a row's maximum,
// one for its sum), so a slot is written again only after a later barrier has been passed by every reader.
template<bool IS_MAX>
__device__ __forceinline__ float cta_reduce_alt(float v, float *slot) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    if (nwarps == 1) return v;
    if (lane == 0) slot[warp] = v;
    __syncthreads();
    float r = slot[0];
    for (int w = 1; w < nwarps; ++w) r = IS_MAX ? fmaxf(r, slot[w]) : r + slot[w];
    return r;
}

// ---- thread-block clusters: one row spread over up to 8 CTAs ------------------------------------------------
// Rank of this CTA in its cluster / number of CTAs per cluster (1 when the launch carries no cluster dimension).
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// Hardware barrier over all threads of all CTAs of the cluster (release / acquire: shared-memory writes made
// before it are visible to distributed-shared-memory reads made after it).  Cannot hang: every thread of every
// CTA of a cluster reaches it, the kernels below have no early exit.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Reads a float from the same shared-memory variable of CTA `rank` of the cluster.
__device__ __forceinline__ float ld_dsmem_f32(const float *local, uint32_t rank) {
    const uint32_t a = (uint32_t) __cvta_generic_to_shared(local);
    uint32_t ra;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
    return v;
}

// Cluster-wide reduction for kernels that give a whole cluster (cl CTAs, a power of two up to 8) to a row:
// the CTA-wide result goes to `*mine` (one float of shared memory per reduction of a row, not reused before the
// row's closing cluster_sync_all), one cluster barrier, then lane r of every warp fetches CTA r's part over
// distributed shared memory and a butterfly over the first cl lanes combines them in the same order everywhere,
// so every thread of the cluster holds the same bits.  All threads of the cluster must call it.
template<bool IS_MAX>
__device__ __forceinline__ float cluster_reduce(float v, float *slot, float *mine, uint32_t cl) {
    v = cta_reduce_alt<IS_MAX>(v, slot);
    if (threadIdx.x == 0) *mine = v;
    cluster_sync_all();
    const uint32_t lane = threadIdx.x & 31;
    float p = ld_dsmem_f32(mine, lane < cl ? lane : 0);
    for (uint32_t o = cl >> 1; o > 0; o >>= 1) {
        const float q = __shfl_xor_sync(0xffffffffu, p, o);
        p = IS_MAX ? fmaxf(p, q) : p + q;
    }
    return __shfl_sync(0xffffffffu, p, 0);
}

// One-dimensional launch with `cl` consecutive CTAs forming a cluster (grid must be a multiple of cl).
template<typename... KArgs, typename... Args>
static inline cudaError_t launch_cluster_smem(void (*kernel)(KArgs...), uint32_t grid, uint32_t threads, uint32_t cl,
                                              size_t smem_bytes, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template<typename... KArgs, typename... Args>
static inline cudaError_t launch_cluster(void (*kernel)(KArgs...), uint32_t grid, uint32_t threads, uint32_t cl,
                                         cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Does a block of `threads` threads of this kernel fit the SM's 65536 registers?  (Kernels without a launch bound
// are compiled with whatever register count serves them best; the launch shapes are checked against it here
// instead of trusting a table.)  One query per kernel and process.
template<auto Kernel>
static inline bool fits_register_file(uint32_t threads) {
    static const int regs = [] {
        cudaFuncAttributes a;
        if (cudaFuncGetAttributes(&a, Kernel) != cudaSuccess) {
            cudaGetLastError();
            return 255;
        }
        return a.numRegs;
    }();
    const uint32_t per_thread = ((uint32_t) regs + 7u) / 8u * 8u;// allocation granularity
    return per_thread * ((threads + 31u) / 32u * 32u) <= 65536u;
}

// Shape of a launch that gives each row to one CTA or to one cluster: `cl` CTAs of `threads` threads, each
// thread holding `vpt` 128-bit vectors.  `want_vpt` is the preferred vectors per thread (bytes in flight when
// there are many rows).  One CTA holds rows of up to 4096 vectors (512 threads x 8 or 1024 x 4; measured on
// B200, one CTA is faster than a cluster wherever the row fits one: [8192, 16384] RMSNorm 103 us against 161 us
// with two CTAs per row); longer rows are spread over a cluster of 2, 4 or 8 CTAs of up to 1024 threads with
// four vectors each, i.e. rows of up to 32768 vectors.
struct RowLaunch {
    uint32_t cl, threads;
    int vpt;
};
static inline RowLaunch row_launch_shape(uint32_t vecs, uint32_t want_vpt) {
    RowLaunch r;
    if (vecs <= 4096) {
        r.cl = 1;
        const uint32_t min_vpt = (vecs + 1023) / 1024;
        const uint32_t want = want_vpt < min_vpt ? min_vpt : want_vpt;
        r.vpt = want <= 1 ? 1 : want <= 2 ? 2 : want <= 4 ? 4 : 8;
        r.threads = ((vecs + r.vpt - 1) / r.vpt + 31) / 32 * 32;
        return r;
    }
    const uint32_t ctas = (vecs + 4095) / 4096;
    r.cl = ctas <= 2 ? 2 : ctas <= 4 ? 4 : 8;
    r.vpt = 4;
    const uint32_t per_cta = (vecs + r.cl - 1) / r.cl;
    r.threads = ((per_cta + 3) / 4 + 31) / 32 * 32;
    return r;
}

}// namespace b200
