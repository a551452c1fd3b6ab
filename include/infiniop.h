/*
 * infiniop.h - C ABI of the B200 (sm_100a) backend for the InfiniOperators
 * decode hot path.
 *
 * The library built from operators_b200/csrc exports exactly the symbols the
 * reference's `libinfiniop.so` exports for these operators, with identical
 * argument lists, enum values and struct layouts, so the reference's ctypes
 * wrapper (operatorspy/liboperators.py) and C callers load it unchanged as the
 * `DevNvGpu` device.  Every declaration cites the reference header it
 * replaces (paths relative to the reference project root).
 *
 * Call pattern ("3+1 stages", reference README.md:9-40):
 *   infiniopCreate<Op>Descriptor -> infiniopGet<Op>WorkspaceSize ->
 *   infiniop<Op> (asynchronous on `stream`) -> infiniopDestroy<Op>Descriptor.
 * All data pointers are device pointers on the handle's GPU; `stream` is a
 * cudaStream_t (NULL = legacy default stream).  Nothing allocates device
 * memory inside a compute call; no call synchronises the device.
 */
#ifndef INFINIOP_B200_H
#define INFINIOP_B200_H

#include <stdint.h>

#ifdef __cplusplus
#define INFINIOP_C extern "C"
#else
#define INFINIOP_C
#endif
#if defined(__GNUC__)
#define INFINIOP_EXPORT __attribute__((visibility("default")))
#else
#define INFINIOP_EXPORT
#endif
#define INFINIOP_API INFINIOP_C INFINIOP_EXPORT

/* Names the reference headers use for the same two macros (include/export.h:4-16). */
#ifndef __export
#define __export INFINIOP_EXPORT
#endif
#ifndef __C
#define __C INFINIOP_C
#endif

/* ---- status codes: include/status.h:4-14 ---------------------------------- */
typedef enum {
    STATUS_SUCCESS = 0,
    STATUS_EXECUTION_FAILED = 1,
    STATUS_BAD_PARAM = 2,
    STATUS_BAD_TENSOR_DTYPE = 3,
    STATUS_BAD_TENSOR_SHAPE = 4,
    STATUS_BAD_TENSOR_STRIDES = 5,
    STATUS_MEMORY_NOT_ALLOCATED = 6,
    STATUS_INSUFFICIENT_WORKSPACE = 7,
    STATUS_BAD_DEVICE = 8,
} infiniopStatus_t;

/* ---- device enum: include/device.h:4-9.  Only DevNvGpu is served here. ---- */
enum DeviceEnum {
    DevCpu = 0,
    DevNvGpu = 1,
    DevCambriconMlu = 2,
    DevAscendNpu = 3,
};
typedef enum DeviceEnum Device;

/* ---- data layout: include/data_type.h:4-47 -------------------------------- *
 * A 32-bit bit-field passed BY VALUE; two layouts are equal when their 32-bit
 * images are equal.  Little-endian images: F16 0x050A0501, BF16 0x08070501,
 * F32 0x08170901, U64 0x00401001.
 */
typedef struct DataLayout {
    unsigned short packed : 8, sign : 1, size : 7, mantissa : 8, exponent : 8;
} DataLayout;
typedef struct DataLayout DT;

#define INFINIOP_DT(p, s, z, m, e) {p, s, z, m, e}
static const DataLayout I8 = INFINIOP_DT(1, 1, 1, 7, 0), I16 = INFINIOP_DT(1, 1, 2, 15, 0),
                        I32 = INFINIOP_DT(1, 1, 4, 31, 0), I64 = INFINIOP_DT(1, 1, 8, 63, 0),
                        U8 = INFINIOP_DT(1, 0, 1, 8, 0), U16 = INFINIOP_DT(1, 0, 2, 16, 0),
                        U32 = INFINIOP_DT(1, 0, 4, 32, 0), U64 = INFINIOP_DT(1, 0, 8, 64, 0),
                        F16 = INFINIOP_DT(1, 1, 2, 10, 5), BF16 = INFINIOP_DT(1, 1, 2, 7, 8),
                        F32 = INFINIOP_DT(1, 1, 4, 23, 8), F64 = INFINIOP_DT(1, 1, 8, 52, 11);

/* ---- tensor descriptor: include/tensor.h:7-18 ----------------------------- *
 * Layout is visible to callers (the Python wrapper mirrors it field by field).
 * Strides are in ELEMENTS and may describe a view into a larger buffer.
 */
struct TensorDescriptor {
    DT dt;
    uint64_t ndim;
    uint64_t *shape;
    int64_t *strides;
};
typedef struct TensorDescriptor *infiniopTensorDescriptor_t;

/* include/tensor/tensor_descriptor.h:8-10.  Copies shape and strides;
 * strides == NULL means contiguous row-major; ndim == 0 is legal. */
INFINIOP_API infiniopStatus_t infiniopCreateTensorDescriptor(infiniopTensorDescriptor_t *desc_ptr, uint64_t ndim,
                                                             uint64_t const *shape, int64_t const *strides,
                                                             DataLayout datatype);
INFINIOP_API infiniopStatus_t infiniopDestroyTensorDescriptor(infiniopTensorDescriptor_t desc);

/* ---- handle: include/handle.h:6-10, include/handle/handle_export.h:8-10 --- *
 * The object behind the pointer starts with `Device device`.  Errors:
 * NULL handle_ptr -> MEMORY_NOT_ALLOCATED, device_id < 0 -> BAD_PARAM, a device
 * other than DevNvGpu or a device_id beyond the visible GPUs -> BAD_DEVICE. */
typedef struct HandleStruct {
    Device device;
} HandleStruct;
typedef HandleStruct *infiniopHandle_t;

INFINIOP_API infiniopStatus_t infiniopCreateHandle(infiniopHandle_t *handle_ptr, Device device, int device_id);
INFINIOP_API infiniopStatus_t infiniopDestroyHandle(infiniopHandle_t handle);

/* Every operator descriptor starts with `Device device`
 * (e.g. include/ops/rms_norm/rms_norm.h:7-11); the rest is private. */

/* ---- RMSNorm: include/ops/rms_norm/rms_norm.h:13-26 ----------------------- *
 * y[n,d] = x[n,d] * rsqrt(mean(x^2) + epsilon) * w[d]; y, x fp16 with unit
 * column stride and free row strides, w fp16 or fp32. */
typedef struct RMSNormDescriptor {
    Device device;
} RMSNormDescriptor;
typedef RMSNormDescriptor *infiniopRMSNormDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateRMSNormDescriptor(infiniopHandle_t handle,
                                                              infiniopRMSNormDescriptor_t *desc_ptr,
                                                              infiniopTensorDescriptor_t y_desc,
                                                              infiniopTensorDescriptor_t x_desc,
                                                              infiniopTensorDescriptor_t w_desc, float epsilon);
INFINIOP_API infiniopStatus_t infiniopGetRMSNormWorkspaceSize(infiniopRMSNormDescriptor_t desc, uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopRMSNorm(infiniopRMSNormDescriptor_t desc, void *workspace,
                                              uint64_t workspace_size, void *y, void const *x, void const *w,
                                              void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyRMSNormDescriptor(infiniopRMSNormDescriptor_t desc);

/* ---- RoPE: include/ops/rotary_embedding/rotary_embedding.h:7-30 ----------- *
 * In place on t[tokens, heads, dh] fp16 (unit last stride), rotating adjacent
 * pairs with caller-supplied fp32 sin/cos tables [max_pos, dh] indexed by the
 * u64 position ids.  A NULL data pointer returns STATUS_BAD_PARAM. */
typedef struct RoPEDescriptor RoPEDescriptor;
typedef RoPEDescriptor *infiniopRoPEDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateRoPEDescriptor(infiniopHandle_t handle, infiniopRoPEDescriptor_t *desc_ptr,
                                                           infiniopTensorDescriptor_t t,
                                                           infiniopTensorDescriptor_t pos_ids,
                                                           infiniopTensorDescriptor_t sin_table,
                                                           infiniopTensorDescriptor_t cos_table);
INFINIOP_API infiniopStatus_t infiniopGetRoPEWorkspaceSize(infiniopRoPEDescriptor_t desc, uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopRoPE(infiniopRoPEDescriptor_t desc, void *workspace, uint64_t workspace_size,
                                           void *t, void const *pos_ids, void const *sin_table,
                                           void const *cos_table, void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyRoPEDescriptor(infiniopRoPEDescriptor_t desc);

/* ---- RoPE written to a second view (NO counterpart in the reference) ------- *
 * dst[i, j, :] = the rotation infiniopRoPE applies to src[i, j, :]; src is not
 * modified.  dst and src: fp16 [tokens, heads, dh] views with unit innermost
 * stride and otherwise free strides, so dst can be the rows of a K cache
 * [heads, max_seq, dh] at the tokens' positions.  Bit for bit what infiniopRoPE
 * followed by infiniopRearrange writes (the reference reaches it through
 * include/ops/rotary_embedding/rotary_embedding.h:10-30 and the rearrange of k
 * into k_cache in src/ops/attention/operator.cc:87-91).  dst and src must not
 * overlap. */
typedef struct RoPEDescriptor *infiniopRoPERearrangeDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateRoPERearrangeDescriptor(infiniopHandle_t handle,
                                                                    infiniopRoPERearrangeDescriptor_t *desc_ptr,
                                                                    infiniopTensorDescriptor_t dst,
                                                                    infiniopTensorDescriptor_t src,
                                                                    infiniopTensorDescriptor_t pos_ids,
                                                                    infiniopTensorDescriptor_t sin_table,
                                                                    infiniopTensorDescriptor_t cos_table);
INFINIOP_API infiniopStatus_t infiniopGetRoPERearrangeWorkspaceSize(infiniopRoPERearrangeDescriptor_t desc,
                                                                    uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopRoPERearrange(infiniopRoPERearrangeDescriptor_t desc, void *workspace,
                                                    uint64_t workspace_size, void *dst, void const *src,
                                                    void const *pos_ids, void const *sin_table,
                                                    void const *cos_table, void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyRoPERearrangeDescriptor(infiniopRoPERearrangeDescriptor_t desc);

/* ---- SwiGLU: include/ops/swiglu/swiglu.h:7-25 ----------------------------- *
 * c = a * silu(b), 2-D fp16, unit column stride, free row strides; c may alias
 * a or b.  No workspace entry point exists for this operator. */
typedef struct SwiGLUDescriptor {
    Device device;
} SwiGLUDescriptor;
typedef SwiGLUDescriptor *infiniopSwiGLUDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateSwiGLUDescriptor(infiniopHandle_t handle,
                                                             infiniopSwiGLUDescriptor_t *desc_ptr,
                                                             infiniopTensorDescriptor_t c_desc,
                                                             infiniopTensorDescriptor_t a_desc,
                                                             infiniopTensorDescriptor_t b_desc);
INFINIOP_API infiniopStatus_t infiniopSwiGLU(infiniopSwiGLUDescriptor_t desc, void *c, void const *a, void const *b,
                                             void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroySwiGLUDescriptor(infiniopSwiGLUDescriptor_t desc);

/* ---- Add: include/ops/add/add.h:7-25 -------------------------------------- *
 * c = a + b with numpy-style broadcasting of a and b to c's shape; contiguous
 * fp16 or fp32 tensors; c may alias a or b when nothing is broadcast. */
typedef struct AddDescriptor {
    Device device;
} AddDescriptor;
typedef AddDescriptor *infiniopAddDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateAddDescriptor(infiniopHandle_t handle, infiniopAddDescriptor_t *desc_ptr,
                                                          infiniopTensorDescriptor_t c, infiniopTensorDescriptor_t a,
                                                          infiniopTensorDescriptor_t b);
INFINIOP_API infiniopStatus_t infiniopAdd(infiniopAddDescriptor_t desc, void *c, void const *a, void const *b,
                                          void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyAddDescriptor(infiniopAddDescriptor_t desc);

/* ---- rearrange: include/ops/rearrange/rearrange.h:7-20 --------------------- *
 * dst[..] = src[..] between two views of equal shape and element type whose
 * innermost stride is 1; outer strides are arbitrary.  Bytes are copied, any
 * DataLayout.  Up to 8 dimensions (the reference's nv-gpu code: 3). */
typedef struct RearrangeDescriptor {
    Device device;
} RearrangeDescriptor;
typedef RearrangeDescriptor *infiniopRearrangeDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateRearrangeDescriptor(infiniopHandle_t handle,
                                                                infiniopRearrangeDescriptor_t *desc_ptr,
                                                                infiniopTensorDescriptor_t dst,
                                                                infiniopTensorDescriptor_t src);
INFINIOP_API infiniopStatus_t infiniopRearrange(infiniopRearrangeDescriptor_t desc, void *dst, void const *src,
                                                void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyRearrangeDescriptor(infiniopRearrangeDescriptor_t desc);

/* ---- fused residual add + RMSNorm (NO counterpart in the reference) -------- *
 * sum = a + b as infiniopAdd forms it, y = RMSNorm(sum) * w as infiniopRMSNorm
 * forms it, in one pass: the sum is bit for bit that of infiniopAdd, y is what
 * infiniopRMSNorm makes of it (up to the grouping of the fp32 sum of squares),
 * and the sum is not read back from memory.  y, sum, a, b: 2-D fp16 of one shape, unit
 * column stride, free row strides, no broadcasting; w 1-D fp16 or fp32.  `sum`
 * may be `a` or `b` (residual updated in place); `y` must not overlap `sum`.
 * The reference's callers reach the same result through
 * include/ops/add/add.h:13-25 followed by include/ops/rms_norm/rms_norm.h:13-26. */
typedef struct AddRMSNormDescriptor {
    Device device;
} AddRMSNormDescriptor;
typedef AddRMSNormDescriptor *infiniopAddRMSNormDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateAddRMSNormDescriptor(infiniopHandle_t handle,
                                                                 infiniopAddRMSNormDescriptor_t *desc_ptr,
                                                                 infiniopTensorDescriptor_t y_desc,
                                                                 infiniopTensorDescriptor_t sum_desc,
                                                                 infiniopTensorDescriptor_t a_desc,
                                                                 infiniopTensorDescriptor_t b_desc,
                                                                 infiniopTensorDescriptor_t w_desc, float epsilon);
INFINIOP_API infiniopStatus_t infiniopGetAddRMSNormWorkspaceSize(infiniopAddRMSNormDescriptor_t desc, uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopAddRMSNorm(infiniopAddRMSNormDescriptor_t desc, void *workspace,
                                                 uint64_t workspace_size, void *y, void *sum, void const *a,
                                                 void const *b, void const *w, void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyAddRMSNormDescriptor(infiniopAddRMSNormDescriptor_t desc);

/* ---- attention: include/ops/attention/attention.h:9-37 --------------------- *
 * k, v[n_kv_head, seq, dh] are written to k_cache, v_cache[n_kv_head, buf, dh]
 * at rows pos .. pos+seq; out[seq, n_q_head, dh] (contiguous) = causal attention
 * of q[n_q_head, seq, dh] over rows 0 .. pos+seq of the caches, scores scaled
 * by 1/sqrt(dh).  fp16, unit innermost strides, dh <= 256.  `pos` is part of
 * the descriptor, as in the reference.  The workspace must hold the reported
 * size, else STATUS_MEMORY_NOT_ALLOCATED. */
typedef struct AttentionDescriptor {
    Device device;
} AttentionDescriptor;
typedef AttentionDescriptor *infiniopAttentionDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateAttentionDescriptor(infiniopHandle_t handle,
                                                                infiniopAttentionDescriptor_t *desc_ptr,
                                                                infiniopTensorDescriptor_t out_desc,
                                                                infiniopTensorDescriptor_t q_desc,
                                                                infiniopTensorDescriptor_t k_desc,
                                                                infiniopTensorDescriptor_t v_desc,
                                                                infiniopTensorDescriptor_t k_cache_desc,
                                                                infiniopTensorDescriptor_t v_cache_desc, uint64_t pos);
INFINIOP_API infiniopStatus_t infiniopGetAttentionWorkspaceSize(infiniopAttentionDescriptor_t desc, uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopAttention(infiniopAttentionDescriptor_t desc, void *workspace,
                                                uint64_t workspace_size, void *out, void const *q, void const *k,
                                                void const *v, void *k_cache, void *v_cache, void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyAttentionDescriptor(infiniopAttentionDescriptor_t desc);

/* ---- matmul: include/ops/matmul/matmul.h:7-32 ------------------------------ *
 * c = alpha * a b + beta * c on 2-D [m,k] x [k,n] or batched 3-D matrices,
 * fp16 or fp32, each matrix with one unit stride (src/ops/matmul/blas.h:9-113);
 * a and b may have batch 1 against a batched c.  fp32 accumulation. */
typedef struct MatmulDescriptor {
    Device device;
} MatmulDescriptor;
typedef MatmulDescriptor *infiniopMatmulDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateMatmulDescriptor(infiniopHandle_t handle,
                                                             infiniopMatmulDescriptor_t *desc_ptr,
                                                             infiniopTensorDescriptor_t c_desc, float alpha,
                                                             infiniopTensorDescriptor_t a_desc,
                                                             infiniopTensorDescriptor_t b_desc, float beta);
INFINIOP_API infiniopStatus_t infiniopGetMatmulWorkspaceSize(infiniopMatmulDescriptor_t desc, uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopMatmul(infiniopMatmulDescriptor_t desc, void *workspace, uint64_t workspace_size,
                                             void *c, void const *a, void const *b, void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyMatmulDescriptor(infiniopMatmulDescriptor_t desc);

/* ---- MLP: include/ops/mlp/mlp.h:9-38 ----------------------------------------- *
 * y = (residual ? y : 0) + alpha * SwiGLU(x w12) w3 with x, y [tokens, hidden],
 * w12 [hidden, 2 * intermediate] holding the gate columns first and the up
 * columns second, w3 [intermediate, hidden] (src/ops/mlp/operator.cc:22-122).
 * fp16; x and y need a unit last stride.  The workspace must hold the reported
 * size, else STATUS_MEMORY_NOT_ALLOCATED. */
typedef struct MLPDescriptor {
    Device device;
} MLPDescriptor;
typedef MLPDescriptor *infiniopMLPDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateMLPDescriptor(infiniopHandle_t handle, infiniopMLPDescriptor_t *desc_ptr,
                                                          infiniopTensorDescriptor_t y_desc,
                                                          infiniopTensorDescriptor_t x_desc,
                                                          infiniopTensorDescriptor_t w12_desc,
                                                          infiniopTensorDescriptor_t w3_desc, float alpha,
                                                          char residual);
INFINIOP_API infiniopStatus_t infiniopGetMLPWorkspaceSize(infiniopMLPDescriptor_t desc, uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopMLP(infiniopMLPDescriptor_t desc, void *workspace, uint64_t workspace_size,
                                          void *y, void const *x, void const *w12, void const *w3, void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyMLPDescriptor(infiniopMLPDescriptor_t desc);

/* ---- causal softmax: include/ops/causal_softmax/causal_softmax.h:7-25 ----- *
 * In place on fp16 [.., seq_len, total_seq_len] (2-D or 3-D, unit last
 * stride): row i keeps columns j <= total_seq_len - seq_len + i, the rest
 * become exact zeros. */
typedef struct CausalSoftmaxDescriptor {
    Device device;
} CausalSoftmaxDescriptor;
typedef CausalSoftmaxDescriptor *infiniopCausalSoftmaxDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateCausalSoftmaxDescriptor(infiniopHandle_t handle,
                                                                    infiniopCausalSoftmaxDescriptor_t *desc_ptr,
                                                                    infiniopTensorDescriptor_t y_desc);
INFINIOP_API infiniopStatus_t infiniopGetCausalSoftmaxWorkspaceSize(infiniopCausalSoftmaxDescriptor_t desc,
                                                                    uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopCausalSoftmax(infiniopCausalSoftmaxDescriptor_t desc, void *workspace,
                                                    uint64_t workspace_size, void *data, void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyCausalSoftmaxDescriptor(infiniopCausalSoftmaxDescriptor_t desc);

/* ---- random sample: include/ops/random_sample/random_sample.h:7-28 -------- *
 * probs: 1-D fp16 logits [voc]; result: u64 [1].  topp > 0 && topk > 1 selects
 * temperature / top-k / top-p sampling driven by the uniform draw random_val,
 * otherwise argmax.  The sampled index follows the reference's CPU backend. */
typedef struct RandomSampleDescriptor {
    Device device;
} RandomSampleDescriptor;
typedef RandomSampleDescriptor *infiniopRandomSampleDescriptor_t;
INFINIOP_API infiniopStatus_t infiniopCreateRandomSampleDescriptor(infiniopHandle_t handle,
                                                                   infiniopRandomSampleDescriptor_t *desc_ptr,
                                                                   infiniopTensorDescriptor_t result,
                                                                   infiniopTensorDescriptor_t probs);
INFINIOP_API infiniopStatus_t infiniopGetRandomSampleWorkspaceSize(infiniopRandomSampleDescriptor_t desc,
                                                                   uint64_t *size);
INFINIOP_API infiniopStatus_t infiniopRandomSample(infiniopRandomSampleDescriptor_t desc, void *workspace,
                                                   uint64_t workspace_size, void *result, void const *probs,
                                                   float random_val, float topp, int topk, float temperature,
                                                   void *stream);
INFINIOP_API infiniopStatus_t infiniopDestroyRandomSampleDescriptor(infiniopRandomSampleDescriptor_t desc);

#endif /* INFINIOP_B200_H */
