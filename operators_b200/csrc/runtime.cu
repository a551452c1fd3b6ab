// Handle and tensor-descriptor entry points of the C ABI.
//
// Replaces, for the DevNvGpu device only, reference src/devices/handle.cc:16-74
// with src/devices/cuda/cuda_handle.cc:3-47 (no cuBLAS / cuDNN handle pools:
// none of the operators served here calls a library) and
// src/tensor/tensor_descriptor.cc:4-26.
#include "common.cuh"

#include "../../include/infiniop_ext.h"

#include <atomic>
#include <new>

using namespace b200;

namespace {
std::atomic<int> g_kernel_choice[kFamilyCount];
}

int b200::kernel_choice(int family) {
    return family >= 0 && family < kFamilyCount ? g_kernel_choice[family].load(std::memory_order_relaxed) : 0;
}

INFINIOP_API infiniopStatus_t infiniopExtSelectKernel(int family, int variant) {
    if (family < 0 || family >= kFamilyCount || variant < 0) return STATUS_BAD_PARAM;
    g_kernel_choice[family].store(variant, std::memory_order_relaxed);
    return STATUS_SUCCESS;
}

namespace b200 {
unsigned long long rope_pipeline_timeouts_read();
bool rope_pipeline_set_wait_polls(unsigned int polls);
unsigned long long tc_gemm_timeouts_read();
unsigned long long rms_norm_ring_timeouts_read();
unsigned long long causal_softmax_ring_timeouts_read();
unsigned long long attn_fused_timeouts_read();
unsigned long long peer_exchange_timeouts_read();
unsigned long long random_sample_pair_timeouts_read();
}// namespace b200

INFINIOP_API infiniopStatus_t infiniopExtDeviceTimeouts(infiniopHandle_t handle, uint64_t *count) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (count == nullptr) return STATUS_BAD_PARAM;
    DeviceGuard guard(reinterpret_cast<Handle *>(handle)->device_id);
    const unsigned long long parts[7] = {rope_pipeline_timeouts_read(), tc_gemm_timeouts_read(),
                                         rms_norm_ring_timeouts_read(), causal_softmax_ring_timeouts_read(),
                                         attn_fused_timeouts_read(), peer_exchange_timeouts_read(),
                                         random_sample_pair_timeouts_read()};
    unsigned long long sum = 0;
    for (unsigned long long v : parts) {
        if (v == ~0ull) return STATUS_EXECUTION_FAILED;
        sum += v;
    }
    *count = sum;
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopExtSetWaitLimit(infiniopHandle_t handle, uint32_t polls) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    DeviceGuard guard(reinterpret_cast<Handle *>(handle)->device_id);
    return rope_pipeline_set_wait_polls(polls) ? STATUS_SUCCESS : STATUS_EXECUTION_FAILED;
}

INFINIOP_API infiniopStatus_t infiniopCreateHandle(infiniopHandle_t *handle_ptr, Device device, int device_id) {
    if (handle_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (device_id < 0) return STATUS_BAD_PARAM;
    // This library is the nv-gpu device and nothing else: there is no CPU path
    // to fall back to, so every other device is refused.
    if (device != DevNvGpu) return STATUS_BAD_DEVICE;

    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device_id >= count) {
        cudaGetLastError();
        return STATUS_BAD_DEVICE;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_id) != cudaSuccess) return STATUS_BAD_DEVICE;
    if (prop.major < 10) {
        fprintf(stderr, "infiniop[b200]: device %d is sm_%d%d; this build carries sm_100a code only\n", device_id,
                prop.major, prop.minor);
        return STATUS_BAD_DEVICE;
    }
    auto *h = new (std::nothrow) Handle{DevNvGpu, device_id, prop.multiProcessorCount,
                                        (int) prop.sharedMemPerBlockOptin};
    if (h == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    *handle_ptr = reinterpret_cast<infiniopHandle_t>(h);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopDestroyHandle(infiniopHandle_t handle) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    delete reinterpret_cast<Handle *>(handle);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopCreateTensorDescriptor(infiniopTensorDescriptor_t *desc_ptr, uint64_t ndim,
                                                             uint64_t const *shape_, int64_t const *strides_,
                                                             DataLayout datatype) {
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    uint64_t *shape = new (std::nothrow) uint64_t[ndim ? ndim : 1];
    int64_t *strides = new (std::nothrow) int64_t[ndim ? ndim : 1];
    auto *d = new (std::nothrow) TensorDescriptor;
    if (!shape || !strides || !d) {
        delete[] shape;
        delete[] strides;
        delete d;
        return STATUS_MEMORY_NOT_ALLOCATED;
    }
    for (uint64_t i = 0; i < ndim; ++i) shape[i] = shape_[i];
    if (strides_ != nullptr) {
        for (uint64_t i = 0; i < ndim; ++i) strides[i] = strides_[i];
    } else {
        int64_t run = 1;
        for (int64_t i = (int64_t) ndim - 1; i >= 0; --i) {
            strides[i] = run;
            run *= (int64_t) shape[i];
        }
    }
    d->dt = datatype;
    d->ndim = ndim;
    d->shape = shape;
    d->strides = strides;
    *desc_ptr = d;
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopDestroyTensorDescriptor(infiniopTensorDescriptor_t desc) {
    if (desc == nullptr) return STATUS_BAD_PARAM;
    delete[] desc->shape;
    delete[] desc->strides;
    delete desc;
    return STATUS_SUCCESS;
}
