// Planning and launch interface of the matmul kernels, shared by infiniopMatmul and the composites built on it
// (infiniopMLP).  A plan is made once per descriptor from shapes and strides; the data pointers arrive per call.
#pragma once
#include "common.cuh"
#include "tc_gemm.cuh"

#include <mutex>

namespace b200 {

// One matrix of the product as the reference's BlasMatrix sees it (reference src/ops/matmul/blas.h:9-48).
struct MatView {
    uint32_t batch, rows, cols;
    int64_t batch_stride, row_stride, col_stride;// elements; batch_stride 0 = broadcast
    uint32_t batch_div;                          // this matrix's batch index = result batch index / batch_div
};

// A matrix as a tensor-core operand: `rows` x k, K-major (k contiguous) or MN-major (rows contiguous).
struct TcOperand {
    uint32_t rows, k, batch, mn_major;
    int64_t ld;          // elements between consecutive rows (K-major) or consecutive k (MN-major)
    int64_t batch_stride;// 0 = broadcast
    uint32_t batch_div;  // operand batch = result batch / batch_div
};

struct MatmulPlan {
    int device_id, sm_count;
    bool f16; // 16-bit storage (fp16, or bf16 when `bf16` is set); otherwise fp32
    bool bf16;
    MatView a, b, c;
    uint32_t batch, m, n, k;
    float alpha, beta;
    int mode;            // tc::EpilogueMode
    // tensor-core path
    bool use_tc, swapped;// swapped: the MMA computes c^T = b^T a^T
    bool pair;           // 256 x 256 tiles on CTA pairs (cta_group::2)
    TcOperand p, q;
    uint32_t p_box_rows, q_box_rows, grid, smem_bytes;
    int counter_slot;    // slot of library-owned stream-K counters, -1: counters in the workspace
    uint64_t partials_bytes, counters_bytes, workspace_bytes;
    tc::GemmParams g;
};

// Tensor maps of the last pair of operand pointers a descriptor was called with.
struct TcMapCache {
    std::mutex mu;
    bool valid = false;
    const void *p_ptr = nullptr, *q_ptr = nullptr;
    CUtensorMap map_p, map_q;
};

// Checks of reference matmul_cuda.cc:12-20 / blas.h:19-100 and the kernel plan.  `epilogue_mode` kEpiSwiGLUCols:
// b holds [gate | up] column halves and c receives up * silu(gate) ([m, n / 2]; c_desc must then describe that
// result's strides with n columns ignored beyond n / 2).  `b_batch_div` > 1: b has batch(c) / b_batch_div matrices
// and result batch i multiplies with b's matrix i / b_batch_div (grouped attention heads sharing one K or V).
infiniopStatus_t matmul_plan_create(MatmulPlan &plan, const Handle *h, infiniopTensorDescriptor_t c_desc, float alpha,
                                    infiniopTensorDescriptor_t a_desc, infiniopTensorDescriptor_t b_desc, float beta,
                                    int epilogue_mode, uint32_t b_batch_div = 1);
void matmul_plan_destroy(MatmulPlan &plan);
infiniopStatus_t matmul_plan_run(MatmulPlan &plan, TcMapCache &cache, void *workspace, uint64_t workspace_size, void *c,
                                 const void *a, const void *b, cudaStream_t stream);
// Tensor map of an fp16 tensor [batch][outer][inner] (inner contiguous, byte strides multiples of 16) read in boxes of
// 64 x box_outer (x box_batch) elements into 128-byte-swizzled shared memory; elements outside the extents read as zero.
bool tc_encode_tiles_f16(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint64_t batch,
                         uint64_t outer_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_outer, uint32_t box_batch = 1);
// Waits that ran out of time inside the tensor-core kernel since the library was loaded (synchronises).
unsigned long long tc_gemm_timeouts_read();

}// namespace b200
