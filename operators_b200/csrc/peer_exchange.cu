// Row exchange over peer memory for vocabulary-sharded sampling (no counterpart in the reference, which has no
// multi-device code).
//
// Every rank holds the columns [col0_r, col0_r + cols_r) of a [rows, voc] logits matrix and is to sample the whole
// rows [row0, row0 + nrows).  Instead of a collective library, two small kernels move the data over NVLink with plain
// loads and stores to memory that the ranks opened to each other through CUDA IPC (one cudaMalloc'd block per rank:
// flags, results, logits shard):
//   gather   announces "my shard is final" to every peer (one 32-bit flag per pair, release at system scope), then
//            each CTA waits for the flag of the one peer it reads from and copies that peer's columns of one of this
//            rank's rows into the local [nrows, voc] matrix (128-bit volatile loads: peer data is never taken from a
//            stale L1 line);
//   publish  writes this rank's sampled indices into every rank's result array, fences, raises a second flag on
//            every peer and waits until every peer has raised it here: after the kernel all rows' indices are
//            local, and every peer has finished reading this rank's shard, so the shard may be overwritten.
// Flags carry a call counter kept in the block itself, so the kernels take no per-call arguments from the host and
// can be captured in a CUDA graph.  No multicast, no multimem: plain peer loads and stores.
//
// Every wait is bounded by a clock budget (about a second); a wait that runs out counts itself in a device counter
// that infiniopExtDeviceTimeouts reports, the kernel finishes with whatever has arrived, and the call has returned
// STATUS_SUCCESS long before: a host that needs certainty reads the counter.
#include "common.cuh"
#include "random_sample.cuh"

#include <cstring>

using namespace b200;

namespace {

// A block starts with 64 flag words (256 bytes): ready[16], done[16], the call counter, the counter of finished rows of
// the one-launch form (random_sample_pair.cu), padding.  The indices are shared with that kernel (random_sample.cuh).
constexpr uint32_t kMaxRanks = kPeerMaxRanks;
constexpr uint32_t kReady = kPeerReady, kDone = kPeerDone, kCalls = kPeerCalls;
constexpr long long kPeerWaitBudget = 2000ll * 1000 * 1000;// clock64 ticks, about a second
constexpr int kCopyThreads = 256;

__device__ unsigned long long g_peer_timeouts = 0;

struct PeerTable {
    const uint16_t *shard[kMaxRanks];// each rank's [rows, cols_r] logits
    int64_t shard_stride[kMaxRanks]; // elements between its rows
    uint32_t col0[kMaxRanks], cols[kMaxRanks];
    uint32_t *flags[kMaxRanks];      // each rank's flag words
    unsigned long long *results[kMaxRanks];
    uint32_t world, rank;
    uint64_t row0, nrows;
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint16_t ld_volatile_u16(const uint16_t *p) {
    uint16_t v;
    asm volatile("ld.volatile.global.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
    return v;
}

// Until *flag has reached `call` (counters wrap; the difference is what counts).  false: the budget ran out.
__device__ __forceinline__ bool wait_flag(const uint32_t *flag, uint32_t call) {
    const long long t0 = clock64();
    while ((int32_t) (ld_acquire_sys(flag) - call) < 0) {
        if (clock64() - t0 > kPeerWaitBudget) {
            atomicAdd(&g_peer_timeouts, 1ull);
            return false;
        }
    }
    return true;
}

// grid (chunks, max(nrows, 1), world): CTA (c, i, p) copies chunk c of peer p's columns of row row0 + i.
template<bool VEC>
__global__ void __launch_bounds__(kCopyThreads) peer_gather_kernel(const PeerTable t, uint16_t *full, int64_t full_stride) {
    __shared__ int s_ok;
    uint32_t *mine = t.flags[t.rank];
    const uint32_t call = mine[kCalls] + 1;// raised by the publish kernel, which runs after this one
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x < t.world) {
        st_release_sys(&t.flags[threadIdx.x][kReady + t.rank], call);// kernel order: the shard is complete
    }
    if (blockIdx.y >= t.nrows) return;// a rank without rows of its own only announces its shard
    const uint32_t p = blockIdx.z;
    // the own shard is final by stream order; a peer's when its flag has arrived
    if (threadIdx.x == 0) s_ok = p == t.rank || wait_flag(&mine[kReady + p], call) ? 1 : 0;
    __syncthreads();
    if (!s_ok) return;
    const uint16_t *src = t.shard[p] + (int64_t) (t.row0 + blockIdx.y) * t.shard_stride[p];
    uint16_t *dst = full + (int64_t) blockIdx.y * full_stride + t.col0[p];
    if (VEC) {
        const uint32_t vecs = t.cols[p] / 8;
        for (uint32_t v = blockIdx.x * kCopyThreads + threadIdx.x; v < vecs; v += gridDim.x * kCopyThreads) {
            reinterpret_cast<uint4 *>(dst)[v] = ld_volatile_v4(reinterpret_cast<const uint4 *>(src) + v);
        }
    } else {
        for (uint32_t e = blockIdx.x * kCopyThreads + threadIdx.x; e < t.cols[p]; e += gridDim.x * kCopyThreads) {
            dst[e] = ld_volatile_u16(src + e);
        }
    }
}

// One CTA.
__global__ void __launch_bounds__(kCopyThreads) peer_publish_kernel(const PeerTable t, const unsigned long long *picked) {
    uint32_t *mine = t.flags[t.rank];
    const uint32_t call = mine[kCalls] + 1;
    for (uint64_t i = threadIdx.x; i < t.nrows * t.world; i += kCopyThreads) {
        const uint32_t p = (uint32_t) (i / t.nrows);
        const uint64_t r = i - (uint64_t) p * t.nrows;
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(t.results[p] + t.row0 + r), "l"(picked[r]) : "memory");
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < t.world) {
        st_release_sys(&t.flags[threadIdx.x][kDone + t.rank], call);
        wait_flag(&mine[kDone + threadIdx.x], call);
    }
    __syncthreads();
    if (threadIdx.x == 0) mine[kCalls] = call;
}

bool fill_table(PeerTable &t, void *const *shards, const int64_t *strides, const uint64_t *col0, const uint64_t *cols,
                void *const *flags, void *const *results, uint32_t world, uint32_t rank, uint64_t row0, uint64_t nrows) {
    if (world == 0 || world > kMaxRanks || rank >= world || flags == nullptr) return false;
    for (uint32_t r = 0; r < world; ++r) {
        if (flags[r] == nullptr) return false;
        t.flags[r] = reinterpret_cast<uint32_t *>(flags[r]);
        t.shard[r] = shards != nullptr ? reinterpret_cast<const uint16_t *>(shards[r]) : nullptr;
        t.shard_stride[r] = strides != nullptr ? strides[r] : 0;
        t.col0[r] = col0 != nullptr ? (uint32_t) col0[r] : 0;
        t.cols[r] = cols != nullptr ? (uint32_t) cols[r] : 0;
        t.results[r] = results != nullptr ? reinterpret_cast<unsigned long long *>(results[r]) : nullptr;
    }
    t.world = world, t.rank = rank, t.row0 = row0, t.nrows = nrows;
    return true;
}

}// namespace

namespace b200 {
unsigned long long peer_exchange_timeouts_read() {
    unsigned long long v = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_timeouts, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return ~0ull;
    }
    return v;
}
}// namespace b200

INFINIOP_API infiniopStatus_t infiniopExtPeerAlloc(infiniopHandle_t handle, uint64_t bytes, void **ptr, unsigned char *ipc_handle) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (ptr == nullptr || ipc_handle == nullptr || bytes == 0) return STATUS_BAD_PARAM;
    DeviceGuard guard(reinterpret_cast<Handle *>(handle)->device_id);
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return STATUS_MEMORY_NOT_ALLOCATED;
    }
    cudaIpcMemHandle_t h;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return STATUS_EXECUTION_FAILED;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the interface carries the handle as 64 bytes");
    memcpy(ipc_handle, &h, sizeof(h));
    *ptr = p;
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopExtPeerOpen(infiniopHandle_t handle, const unsigned char *ipc_handle, void **ptr) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (ptr == nullptr || ipc_handle == nullptr) return STATUS_BAD_PARAM;
    DeviceGuard guard(reinterpret_cast<Handle *>(handle)->device_id);
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle, sizeof(h));
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return STATUS_EXECUTION_FAILED;
    }
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopExtPeerClose(infiniopHandle_t handle, void *ptr) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (ptr == nullptr) return STATUS_SUCCESS;
    DeviceGuard guard(reinterpret_cast<Handle *>(handle)->device_id);
    if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) {
        cudaGetLastError();
        return STATUS_EXECUTION_FAILED;
    }
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopExtPeerFree(infiniopHandle_t handle, void *ptr) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (ptr == nullptr) return STATUS_SUCCESS;
    DeviceGuard guard(reinterpret_cast<Handle *>(handle)->device_id);
    if (cudaFree(ptr) != cudaSuccess) {
        cudaGetLastError();
        return STATUS_EXECUTION_FAILED;
    }
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopExtPeerGatherRows(infiniopHandle_t handle, void *full, int64_t full_row_stride,
                                                        void *const *shards, const int64_t *shard_row_strides,
                                                        const uint64_t *shard_col0, const uint64_t *shard_cols,
                                                        void *const *flags, uint32_t world, uint32_t rank, uint64_t row0,
                                                        uint64_t nrows, void *stream) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    PeerTable t{};
    if (shards == nullptr || shard_row_strides == nullptr || shard_col0 == nullptr || shard_cols == nullptr ||
        !fill_table(t, shards, shard_row_strides, shard_col0, shard_cols, flags, nullptr, world, rank, row0, nrows)) {
        return STATUS_BAD_PARAM;
    }
    if (nrows > 0 && full == nullptr) return STATUS_BAD_PARAM;
    if (nrows > 65535) return STATUS_BAD_PARAM;
    bool vec = full_row_stride % 8 == 0 && aligned16(full);
    uint32_t most = 0;
    for (uint32_t r = 0; r < world; ++r) {
        if (t.shard[r] == nullptr) return STATUS_BAD_PARAM;
        vec = vec && t.cols[r] % 8 == 0 && t.col0[r] % 8 == 0 && t.shard_stride[r] % 8 == 0 && aligned16(t.shard[r]);
        most = t.cols[r] > most ? t.cols[r] : most;
    }
    DeviceGuard guard(reinterpret_cast<Handle *>(handle)->device_id);
    const uint32_t per_cta = kCopyThreads * (vec ? 8 : 1) * 4;// four units per thread
    uint32_t chunks = (most + per_cta - 1) / per_cta;
    chunks = chunks < 1 ? 1 : (chunks > 64 ? 64 : chunks);
    const dim3 grid(chunks, nrows > 0 ? (uint32_t) nrows : 1, world);
    auto st = reinterpret_cast<cudaStream_t>(stream);
    if (vec) peer_gather_kernel<true><<<grid, kCopyThreads, 0, st>>>(t, reinterpret_cast<uint16_t *>(full), full_row_stride);
    else peer_gather_kernel<false><<<grid, kCopyThreads, 0, st>>>(t, reinterpret_cast<uint16_t *>(full), full_row_stride);
    return check_launch("peer gather");
}

INFINIOP_API infiniopStatus_t infiniopExtPeerPublishResults(infiniopHandle_t handle, void *const *results, const void *picked,
                                                            void *const *flags, uint32_t world, uint32_t rank,
                                                            uint64_t row0, uint64_t nrows, void *stream) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    PeerTable t{};
    if (results == nullptr || !fill_table(t, nullptr, nullptr, nullptr, nullptr, flags, results, world, rank, row0, nrows)) {
        return STATUS_BAD_PARAM;
    }
    for (uint32_t r = 0; r < world; ++r) {
        if (t.results[r] == nullptr) return STATUS_BAD_PARAM;
    }
    if (nrows > 0 && picked == nullptr) return STATUS_BAD_PARAM;
    DeviceGuard guard(reinterpret_cast<Handle *>(handle)->device_id);
    peer_publish_kernel<<<1, kCopyThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        t, reinterpret_cast<const unsigned long long *>(picked));
    return check_launch("peer publish");
}
