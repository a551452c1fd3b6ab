// MLP: y = (residual ? y : 0) + alpha * SwiGLU(x w12) w3.
//
// Replaces the composite reference src/ops/mlp/operator.cc:22-122 behind include/ops/mlp/mlp.h.  The reference
// runs three public operators: matmul into a [tokens, 2 * intermediate] workspace, SwiGLU on its two column
// halves into a second workspace, matmul with w3 (beta = 1 carries the residual).  Here the first product runs
// with SwiGLU as its epilogue (tc_gemm.cuh, kEpiSwiGLUCols): every tile holds matching gate and up columns side
// by side in tensor memory, both are narrowed to fp16 exactly as the reference's first matmul stores them, and
// only up * silu(gate) reaches memory, so the [tokens, 2 * intermediate] tensor never exists.  Layouts the
// tensor-core path cannot address fall back to the reference's three steps with this library's operators.
#include "matmul.cuh"

#include <new>

using namespace b200;

namespace {

struct MLPDesc {
    Device device;
    int device_id;
    bool fused;
    uint64_t tokens, hidden, di;
    MatmulPlan up, down;     // x w12 (fused: with the SwiGLU epilogue), act w3
    TcMapCache up_maps, down_maps;
    infiniopSwiGLUDescriptor_t swiglu;// unfused form only
    uint64_t act_bytes, gate_up_bytes, scratch_bytes, workspace_bytes;
};

TensorDescriptor make_desc(DataLayout dt, uint64_t *shape, int64_t *strides) { return TensorDescriptor{dt, 2, shape, strides}; }

uint64_t round256(uint64_t v) { return (v + 255) / 256 * 256; }

}// namespace

INFINIOP_API infiniopStatus_t infiniopCreateMLPDescriptor(infiniopHandle_t handle, infiniopMLPDescriptor_t *desc_ptr,
                                                          infiniopTensorDescriptor_t y_desc,
                                                          infiniopTensorDescriptor_t x_desc,
                                                          infiniopTensorDescriptor_t w12_desc,
                                                          infiniopTensorDescriptor_t w3_desc, float alpha,
                                                          char residual) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    if (y_desc == nullptr || x_desc == nullptr || w12_desc == nullptr || w3_desc == nullptr) return STATUS_BAD_PARAM;
    // checks and codes of reference operator.cc:30-36
    if (y_desc->ndim != 2 || x_desc->ndim != 2 || w12_desc->ndim != 2 || w3_desc->ndim != 2) return STATUS_BAD_TENSOR_SHAPE;
    if (x_desc->strides[1] != 1 || y_desc->strides[1] != 1) return STATUS_BAD_TENSOR_STRIDES;
    // (bf16 is an extension of this library: all four tensors bf16; the reference's MLP is fp16)
    if (!dt_eq(x_desc->dt, F16) && !dt_eq(x_desc->dt, BF16)) return STATUS_BAD_TENSOR_DTYPE;
    const DataLayout dt = x_desc->dt;
    const uint64_t tokens = x_desc->shape[0], hidden = x_desc->shape[1], di = w12_desc->shape[1] / 2;
    if (w12_desc->shape[1] % 2 != 0) return STATUS_BAD_TENSOR_SHAPE;

    auto *h = reinterpret_cast<Handle *>(handle);
    auto *d = new (std::nothrow) MLPDesc{};
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    d->device = DevNvGpu, d->device_id = h->device_id;
    d->tokens = tokens, d->hidden = hidden, d->di = di;
    d->swiglu = nullptr;
    d->up.counter_slot = d->down.counter_slot = -1;

    uint64_t act_shape[2] = {tokens, di};
    int64_t act_strides[2] = {(int64_t) di, 1};
    TensorDescriptor act = make_desc(dt, act_shape, act_strides);
    infiniopStatus_t s = matmul_plan_create(d->up, h, &act, 1.0f, x_desc, w12_desc, 0.0f, tc::kEpiSwiGLUCols);
    d->fused = s == STATUS_SUCCESS && d->up.use_tc;
    d->act_bytes = round256(tokens * di * 2);
    d->gate_up_bytes = 0;
    if (!d->fused) {
        matmul_plan_destroy(d->up);
        // the reference's three steps: [tokens, 2 di], SwiGLU on its halves (operator.cc:38-57)
        uint64_t gu_shape[2] = {tokens, 2 * di};
        int64_t gu_strides[2] = {(int64_t) (2 * di), 1};
        TensorDescriptor gu = make_desc(dt, gu_shape, gu_strides);
        s = matmul_plan_create(d->up, h, &gu, 1.0f, x_desc, w12_desc, 0.0f, tc::kEpiPlain);
        if (s == STATUS_SUCCESS) {
            TensorDescriptor half = make_desc(dt, act_shape, gu_strides);
            s = infiniopCreateSwiGLUDescriptor(handle, &d->swiglu, &act, &half, &half);
        }
        d->gate_up_bytes = round256(tokens * 2 * di * 2);
    }
    if (s == STATUS_SUCCESS) {
        s = matmul_plan_create(d->down, h, y_desc, alpha, &act, w3_desc, residual ? 1.0f : 0.0f, tc::kEpiPlain);
    }
    if (s != STATUS_SUCCESS) {
        if (d->swiglu != nullptr) infiniopDestroySwiGLUDescriptor(d->swiglu);
        matmul_plan_destroy(d->up);
        matmul_plan_destroy(d->down);
        delete d;
        return s;
    }
    d->scratch_bytes = d->up.workspace_bytes > d->down.workspace_bytes ? d->up.workspace_bytes : d->down.workspace_bytes;
    d->workspace_bytes = d->act_bytes + d->gate_up_bytes + d->scratch_bytes + 256;
    *desc_ptr = reinterpret_cast<infiniopMLPDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetMLPWorkspaceSize(infiniopMLPDescriptor_t desc, uint64_t *size) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = reinterpret_cast<MLPDesc *>(desc)->workspace_bytes;
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopMLP(infiniopMLPDescriptor_t desc, void *workspace, uint64_t workspace_size, void *y,
                                          void const *x, void const *w12, void const *w3, void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (y == nullptr || x == nullptr || w12 == nullptr || w3 == nullptr) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<MLPDesc *>(desc);
    if (d->tokens == 0 || d->hidden == 0) return STATUS_SUCCESS;
    if (workspace == nullptr || workspace_size < d->workspace_bytes) return STATUS_MEMORY_NOT_ALLOCATED;// operator.cc:102-104
    DeviceGuard guard(d->device_id);
    auto st = reinterpret_cast<cudaStream_t>(stream);
    unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t) 255);
    void *act = base, *gate_up = base + d->act_bytes, *scratch = base + d->act_bytes + d->gate_up_bytes;
    infiniopStatus_t s;
    if (d->fused) {
        s = matmul_plan_run(d->up, d->up_maps, scratch, d->scratch_bytes, act, x, w12, st);
        if (s != STATUS_SUCCESS) return s;
    } else {
        s = matmul_plan_run(d->up, d->up_maps, scratch, d->scratch_bytes, gate_up, x, w12, st);
        if (s != STATUS_SUCCESS) return s;
        // gate = columns [0, di), up = columns [di, 2 di): c = up * silu(gate) (operator.cc:106-110)
        s = infiniopSwiGLU(d->swiglu, act, reinterpret_cast<uint16_t *>(gate_up) + d->di, gate_up, stream);
        if (s != STATUS_SUCCESS) return s;
    }
    return matmul_plan_run(d->down, d->down_maps, scratch, d->scratch_bytes, y, act, w3, st);
}

INFINIOP_API infiniopStatus_t infiniopDestroyMLPDescriptor(infiniopMLPDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    auto *d = reinterpret_cast<MLPDesc *>(desc);
    if (d->swiglu != nullptr) infiniopDestroySwiGLUDescriptor(d->swiglu);
    matmul_plan_destroy(d->up);
    matmul_plan_destroy(d->down);
    delete d;
    return STATUS_SUCCESS;
}
