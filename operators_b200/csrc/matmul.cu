// Matmul: c = alpha * a b + beta * c on 2-D or batched 3-D fp16 / fp32 matrices with one unit stride each.
//
// Replaces reference src/ops/matmul/cuda/matmul_cuda.cu:8-77 (a cublasGemmStridedBatchedEx call) and
// src/ops/matmul/cuda/matmul_cuda.cc:5-43 behind include/ops/matmul/matmul.h; the layout rules are those of
// src/ops/matmul/blas.h:9-113 (2-D or 3-D, one of the two strides of every matrix must be 1, a and b may be
// broadcast over the batch).  Numerics follow the CPU backend (src/ops/matmul/cpu/matmul_cpu.cc:44-79): fp32
// accumulation over k, then `alpha * sum` (beta == 0) or `beta * c + alpha * sum` in un-fused fp32 and, for fp16,
// the reference's truncating conversion.  Only the order of the fp32 sum over k differs.
//
// fp16 products whose operands a TMA descriptor can address (16-byte aligned bases, leading dimensions that are
// multiples of 8 elements) run on the tensor cores (tc_gemm.cuh: tcgen05.mma, TMEM accumulators, TMA loads).
// Products with at most 64 rows run transposed, so that the other matrix's columns fill the 128 MMA rows and the
// few rows of `a` take 16 .. 64 MMA columns: decoding shapes stream the weight matrix once at HBM speed.
// Everything else (fp32, unaligned layouts) takes a CUDA-core kernel with the same arithmetic.
#define B200_TC_GEMM_KERNEL
#include "matmul.cuh"

#include "../../include/infiniop_ext.h"

#include <atomic>
#include <mutex>
#include <new>

using namespace b200;

namespace {

// ---- CUDA-core kernel: any strides, fp16 or fp32 storage, fp32 accumulation ------------------------------
template<int DT, typename T>
__device__ __forceinline__ float load_elem(const T *p) {
    if constexpr (sizeof(T) == 2) return load16<DT>(*p);
    else return *p;
}

constexpr int kSimtTile = 64, kSimtK = 16;

template<typename T, int DT>
__global__ void __launch_bounds__(256)
    matmul_simt_kernel(T *c, const T *a, const T *b, MatView vc, MatView va, MatView vb, uint32_t m, uint32_t n,
                       uint32_t k, float alpha, float beta) {
    __shared__ float sa[kSimtK][kSimtTile + 1], sb[kSimtK][kSimtTile + 1];
    const uint32_t batch = blockIdx.z;
    const uint32_t m0 = blockIdx.y * kSimtTile, n0 = blockIdx.x * kSimtTile;
    const T *ab = a + (int64_t) (batch / va.batch_div) * va.batch_stride, *bb = b + (int64_t) (batch / vb.batch_div) * vb.batch_stride;
    T *cb = c + (int64_t) batch * vc.batch_stride;
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;// thread computes rows ty*4.., columns tx*4..
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < k; k0 += kSimtK) {
        // 64 x 16 elements of a and 16 x 64 of b: 1024 each, four per thread; the faster index follows the unit stride
        for (uint32_t e = threadIdx.x; e < kSimtTile * kSimtK; e += 256) {
            uint32_t r, kk;
            if (va.col_stride == 1) kk = e % kSimtK, r = e / kSimtK;
            else r = e % kSimtTile, kk = e / kSimtTile;
            float v = 0.f;
            if (m0 + r < m && k0 + kk < k) v = load_elem<DT>(ab + (int64_t) (m0 + r) * va.row_stride + (int64_t) (k0 + kk) * va.col_stride);
            sa[kk][r] = v;
            uint32_t cn, kb;
            if (vb.col_stride == 1) cn = e % kSimtTile, kb = e / kSimtTile;
            else kb = e % kSimtK, cn = e / kSimtK;
            v = 0.f;
            if (n0 + cn < n && k0 + kb < k) v = load_elem<DT>(bb + (int64_t) (k0 + kb) * vb.row_stride + (int64_t) (n0 + cn) * vb.col_stride);
            sb[kb][cn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kSimtK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i], bv[i] = sb[kk][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t r = m0 + ty * 4 + i, cn = n0 + tx * 4 + j;
            if (r < m && cn < n) {
                T *dst = cb + (int64_t) r * vc.row_stride + (int64_t) cn * vc.col_stride;
                float v = __fmul_rn(alpha, acc[i][j]);
                if (beta != 0.f) v = __fadd_rn(__fmul_rn(beta, load_elem<DT>(dst)), v);
                if constexpr (sizeof(T) == 2) *dst = store16<DT>(v);
                else *dst = v;
            }
        }
    }
}

// ---- tensor maps --------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return (EncodeTiledFn) nullptr;
        }
        return (EncodeTiledFn) p;
    }();
    return fn;
}

// One operand seen as rows x k (fp16): K-major when k is contiguous, MN-major when the rows are.
bool encode_operand(CUtensorMap *map, const void *base, const TcOperand &o, uint32_t box_rows, bool bf16) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    // leading dimension in bytes; a dimension of extent 1 gets any legal stride
    const uint64_t inner = o.mn_major ? o.rows : o.k, outer = o.mn_major ? o.k : o.rows;
    uint64_t ld_bytes = (uint64_t) o.ld * 2;
    if (outer == 1 || ld_bytes == 0) ld_bytes = (inner * 2 + 15) / 16 * 16;
    uint64_t batch_bytes = (uint64_t) o.batch_stride * 2;
    if (o.batch <= 1 || batch_bytes == 0) batch_bytes = ld_bytes * outer;
    cuuint64_t dims[3] = {inner, outer, o.batch_stride == 0 ? 1u : o.batch};
    cuuint64_t strides[2] = {ld_bytes, batch_bytes};
    cuuint32_t box[3] = {64, o.mn_major ? 64u : box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                          const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool operand_from_view(TcOperand &o, const MatView &v, bool rows_are_view_rows, uint32_t batch) {
    // the operand's row index is the view's row index (a as P / Q) or its column index (b: rows = n, k = view rows)
    const uint32_t rows = rows_are_view_rows ? v.rows : v.cols, k = rows_are_view_rows ? v.cols : v.rows;
    const int64_t row_stride = rows_are_view_rows ? v.row_stride : v.col_stride;
    const int64_t k_stride = rows_are_view_rows ? v.col_stride : v.row_stride;
    o.rows = rows, o.k = k, o.batch = v.batch, o.batch_stride = v.batch > 1 ? v.batch_stride : 0;
    o.batch_div = v.batch_div;
    (void) batch;
    if (k_stride == 1 && (rows == 1 || (row_stride % 8 == 0 && row_stride >= (int64_t) k))) {
        o.mn_major = 0, o.ld = row_stride;
    } else if (row_stride == 1 && (k == 1 || (k_stride % 8 == 0 && k_stride >= (int64_t) rows))) {
        o.mn_major = 1, o.ld = k_stride;
    } else {
        return false;// a TMA descriptor needs leading dimensions that are multiples of 16 bytes
    }
    return o.batch_stride % 8 == 0 && o.batch_stride >= 0;
}

// ---- stream-K tile counters -----------------------------------------------------------------------------
// A descriptor whose product is split over k keeps one arrival counter per tile.  They live in an array inside
// the library image (zero at load; the CTA that arrives last on a tile puts its counter back to zero), a slot of
// kSlotCounters per descriptor, so that a call needs no launch to clear them.  When all slots are taken, the
// counters go to the caller's workspace and are cleared by a memset before every launch.  A kernel that gave up
// on a wait (see tc_gemm.cuh) can leave counters behind: infiniopExtDeviceTimeouts reports that.
constexpr uint32_t kCounterSlots = 1024, kSlotCounters = 320;
static __device__ uint32_t g_streamk_counters[kCounterSlots * kSlotCounters];
std::mutex g_slot_mu;
bool g_slot_used[kCounterSlots];
std::atomic<uint32_t *> g_counter_pool[64];// device address per device ordinal

int counter_slot_acquire() {
    std::lock_guard<std::mutex> lock(g_slot_mu);
    for (uint32_t i = 0; i < kCounterSlots; ++i) {
        if (!g_slot_used[i]) {
            g_slot_used[i] = true;
            return (int) i;
        }
    }
    return -1;
}
void counter_slot_release(int slot) {
    std::lock_guard<std::mutex> lock(g_slot_mu);
    if (slot >= 0 && slot < (int) kCounterSlots) g_slot_used[slot] = false;
}
// With the descriptor's device current.
uint32_t *counter_pool_address(int device) {
    if (device < 0 || device >= 64) return nullptr;
    uint32_t *p = g_counter_pool[device].load(std::memory_order_acquire);
    if (p == nullptr) {
        void *addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_streamk_counters) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        p = reinterpret_cast<uint32_t *>(addr);
        g_counter_pool[device].store(p, std::memory_order_release);
    }
    return p;
}

}// namespace

namespace b200 {

bool tc_encode_tiles_f16(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint64_t batch,
                         uint64_t outer_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_outer, uint32_t box_batch) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[3] = {inner, outer, batch};
    cuuint64_t strides[2] = {outer_stride_bytes, batch_stride_bytes};
    cuuint32_t box[3] = {64, box_outer, box_batch};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

infiniopStatus_t matmul_plan_create(MatmulPlan &pl, const Handle *h, infiniopTensorDescriptor_t c_desc, float alpha,
                                    infiniopTensorDescriptor_t a_desc, infiniopTensorDescriptor_t b_desc, float beta,
                                    int epilogue_mode, uint32_t b_batch_div) {
    if (c_desc == nullptr || a_desc == nullptr || b_desc == nullptr) return STATUS_BAD_PARAM;
    // dtype first, then the layout checks in the reference's order a, b, c (matmul_cuda.cc:12-20, blas.h:19-48)
    // (bf16 is an extension of this library: the reference's matmul takes fp16 and fp32)
    const bool bf16 = dt_eq(c_desc->dt, BF16);
    const bool f16 = dt_eq(c_desc->dt, F16) || bf16, f32 = dt_eq(c_desc->dt, F32);
    if (!f16 && !f32) return STATUS_BAD_TENSOR_DTYPE;
    infiniopTensorDescriptor_t descs[3] = {a_desc, b_desc, c_desc};
    MatView views[3];
    for (int i = 0; i < 3; ++i) {
        infiniopTensorDescriptor_t t = descs[i];
        MatView &v = views[i];
        v.batch_div = 1;
        if (t->ndim == 2) {
            v.batch = 1, v.batch_stride = 0;
            v.rows = (uint32_t) t->shape[0], v.cols = (uint32_t) t->shape[1];
            v.row_stride = t->strides[0], v.col_stride = t->strides[1];
        } else if (t->ndim == 3) {
            v.batch = (uint32_t) t->shape[0];
            v.batch_stride = v.batch == 1 ? 0 : t->strides[0];
            v.rows = (uint32_t) t->shape[1], v.cols = (uint32_t) t->shape[2];
            v.row_stride = t->strides[1], v.col_stride = t->strides[2];
        } else {
            return STATUS_BAD_TENSOR_SHAPE;
        }
        if (t->shape[t->ndim - 1] > 0x7FFFFFFFull || t->shape[t->ndim - 2] > 0x7FFFFFFFull) return STATUS_BAD_TENSOR_SHAPE;
        if (v.row_stride != 1 && v.col_stride != 1) return STATUS_BAD_TENSOR_STRIDES;
    }
    const MatView &va = views[0], &vb = views[1], &vc = views[2];
    // the reference asserts these (blas.h:86-88); a status code is friendlier than an abort
    const bool swiglu = epilogue_mode == tc::kEpiSwiGLUCols;// c holds up * silu(gate): half of b's columns
    if (swiglu && vb.cols % 2 != 0) return STATUS_BAD_TENSOR_SHAPE;
    if (vc.rows != va.rows || vc.cols != (swiglu ? vb.cols / 2 : vb.cols) || va.cols != vb.rows) return STATUS_BAD_TENSOR_SHAPE;
    if (b_batch_div > 1) {
        if ((uint64_t) views[1].batch * b_batch_div != vc.batch) return STATUS_BAD_PARAM;
        views[1].batch_div = b_batch_div;
    } else if (!(vb.batch == vc.batch || vb.batch == 1)) {
        return STATUS_BAD_PARAM;
    }
    if (!(va.batch == vc.batch || va.batch == 1)) return STATUS_BAD_PARAM;
    if (!dt_eq(a_desc->dt, c_desc->dt) || !dt_eq(b_desc->dt, c_desc->dt)) return STATUS_BAD_TENSOR_DTYPE;
    if (va.row_stride < 0 || va.col_stride < 0 || vb.row_stride < 0 || vb.col_stride < 0 || vc.row_stride < 0 ||
        vc.col_stride < 0) {
        return STATUS_BAD_TENSOR_STRIDES;
    }

    pl = MatmulPlan{};
    pl.device_id = h->device_id, pl.sm_count = h->sm_count;
    pl.f16 = f16, pl.bf16 = bf16;
    pl.a = va, pl.b = vb, pl.c = vc;
    pl.batch = vc.batch, pl.m = vc.rows, pl.n = vb.cols, pl.k = va.cols;
    pl.alpha = alpha, pl.beta = beta;
    pl.mode = epilogue_mode;
    pl.use_tc = false;
    pl.workspace_bytes = 0;
    pl.counter_slot = -1;
    if (!f16 || pl.m == 0 || pl.n == 0 || pl.k == 0 || pl.batch == 0) return STATUS_SUCCESS;

    // ---- tensor-core plan ---------------------------------------------------------------------------
    TcOperand oa, ob;
    if (!operand_from_view(oa, va, true, pl.batch) || !operand_from_view(ob, vb, false, pl.batch)) return STATUS_SUCCESS;
    const uint32_t n_out = swiglu ? pl.n / 2 : pl.n;// columns of the result
    // few rows: run transposed, the other matrix's columns on the 128 lanes and the rows of `a` on 16 .. 64 columns
    pl.swapped = pl.m <= 64 && n_out > pl.m;
    tc::GemmParams &g = pl.g;
    g = tc::GemmParams{};
    pl.p = pl.swapped ? ob : oa;
    pl.q = pl.swapped ? oa : ob;
    g.mode = !swiglu ? tc::kEpiPlain : pl.swapped ? tc::kEpiSwiGLULanes : tc::kEpiSwiGLUCols;
    // the up half starts n_out rows behind the gate half; where that is the operand's contiguous index, a TMA
    // copy can only start there if the offset is a multiple of 16 bytes
    if (swiglu && (pl.swapped ? pl.p.mn_major : pl.q.mn_major) && n_out % 8 != 0) return STATUS_SUCCESS;
    g.mp = pl.p.rows, g.np = pl.q.rows, g.k = pl.k, g.batch = pl.batch;
    g.p_major_mn = pl.p.mn_major, g.q_major_mn = pl.q.mn_major;
    g.bf16 = pl.bf16 ? 1u : 0u;
    g.p_batch_mul = pl.p.batch_stride == 0 ? 0 : 1, g.q_batch_mul = pl.q.batch_stride == 0 ? 0 : 1;
    g.p_batch_div = pl.p.batch_div, g.q_batch_div = pl.q.batch_div;
    g.tiles_m = (g.mp + tc::kBM - 1) / tc::kBM;
    g.p_tiles = 1;
    pl.p_box_rows = tc::kBM;
    const uint32_t gran = g.q_major_mn ? 64u : 16u;// MN-major tiles come in 64-row TMA boxes
    uint32_t bn;
    if (g.mode == tc::kEpiSwiGLUCols) {
        // halves of 64 or 128 columns: 128 + 128 when that still gives every SM two tiles
        const uint32_t tiles128 = g.tiles_m * ((n_out + 127) / 128) * pl.batch;
        const uint32_t half = (n_out >= 128 && tiles128 >= 2u * (uint32_t) pl.sm_count) ? 128u : 64u;
        bn = 2 * half;
        g.tiles_n = (n_out + half - 1) / half;
        g.half_offset = n_out;
        g.np = n_out;
    } else {
        if (g.mode == tc::kEpiSwiGLULanes) {// a tile = 128 features: gate rows and up rows feed two accumulators
            g.mp = n_out, g.half_offset = n_out;
            g.tiles_m = (n_out + tc::kBM - 1) / tc::kBM;
            g.p_tiles = 2;
        }
        const uint32_t np_round = (g.np + gran - 1) / gran * gran;
        bn = np_round < 256 ? np_round : 256;
        if (bn == 256) {// narrower tiles when wide ones would leave SMs without work
            const uint32_t tiles256 = g.tiles_m * ((g.np + 255) / 256) * pl.batch;
            if (tiles256 < 2u * (uint32_t) pl.sm_count) bn = 128;
        }
        g.tiles_n = (g.np + bn - 1) / bn;
    }
    g.bn = bn;
    g.total_tiles = g.tiles_m * g.tiles_n * pl.batch;
    if (g.q_major_mn) {
        g.q_boxes = bn / 64, g.q_box_bytes = 64 * tc::kBK * 2;
        pl.q_box_rows = 64;
    } else if (g.mode == tc::kEpiSwiGLUCols) {
        g.q_boxes = 2, g.q_box_bytes = (bn / 2) * tc::kBK * 2;
        pl.q_box_rows = bn / 2;
    } else {
        g.q_boxes = 1, g.q_box_bytes = bn * tc::kBK * 2;
        pl.q_box_rows = bn;
    }
    const uint32_t q_bytes = g.q_boxes * g.q_box_bytes;
    const uint32_t sub_bytes = g.p_tiles * tc::kPBytes + ((q_bytes + 1023u) & ~1023u);
    const uint32_t budget = (uint32_t) h->max_smem_optin - 8192u;// alignment slack, barriers, the epilogue's hand-over buffer
    // Narrow tiles are weight streaming: four 64-wide k-blocks per pipeline step, so that a step asks for 512
    // contiguous bytes of every weight row at once (measured on [16, 4096] x [4096, 28672]: 51.8 / 51.2 / 48.5 us
    // with one / two / four k-blocks per step)
    g.kbs = bn > 64 ? 1u : budget / (4 * sub_bytes) >= 3 ? 4u : budget / (2 * sub_bytes) >= 3 ? 2u : 1u;
    g.kblocks = (pl.k + tc::kBK * g.kbs - 1) / (tc::kBK * g.kbs);
    const uint32_t stage_bytes = g.kbs * sub_bytes;
    uint32_t stages = budget / stage_bytes;
    if (stages > 10) stages = 10;
    if (stages < 2) return STATUS_SUCCESS;
    g.stages = stages;
    pl.smem_bytes = stages * stage_bytes + 8192;
    // stream-K when whole tiles cannot occupy the GPU twice over
    const uint64_t total_work = (uint64_t) g.total_tiles * g.kblocks;
    g.streamk = g.total_tiles < 2u * (uint32_t) pl.sm_count && g.kblocks >= 2 ? 1u : 0u;
    uint32_t grid = (uint32_t) pl.sm_count;
    if (g.streamk) {
        if (total_work < grid) grid = (uint32_t) total_work;
        g.work_per_cta = (uint32_t) ((total_work + grid - 1) / grid);
        grid = (uint32_t) ((total_work + g.work_per_cta - 1) / g.work_per_cta);
        pl.partials_bytes = (uint64_t) grid * 2ull * tc::kBM * (g.p_tiles * bn) * 4ull;
        pl.counters_bytes = ((uint64_t) g.total_tiles * 4 + 255) / 256 * 256;
        pl.workspace_bytes = pl.partials_bytes + pl.counters_bytes + 256;
        pl.counter_slot = g.total_tiles <= kSlotCounters ? counter_slot_acquire() : -1;
    } else if (g.total_tiles < grid) {
        grid = g.total_tiles;
    }
    pl.grid = grid;
    // Large products: 256 x 256 tiles on CTA pairs (tc_gemm_pair_kernel), when they give every pair at least one tile
    pl.pair = false;
    // (infiniopExtSelectKernel(matmul, 2) at descriptor creation keeps the single-CTA kernel: tests, comparisons)
    if (!pl.swapped && g.mode != tc::kEpiSwiGLULanes && g.mp >= 512 && n_out >= 256 && kernel_choice(kFamilyMatmul) != 2) {
        const uint32_t pairs = (uint32_t) pl.sm_count / 2;
        const uint32_t tm2 = (g.mp + 255) / 256;
        const uint32_t tn2 = g.mode == tc::kEpiSwiGLUCols ? (n_out + 127) / 128 : (g.np + 255) / 256;
        if ((uint64_t) tm2 * tn2 * pl.batch >= pairs) {
            if (pl.counter_slot >= 0) counter_slot_release(pl.counter_slot);
            pl.counter_slot = -1;
            pl.pair = true;
            g.streamk = 0, g.kbs = 1;
            g.kblocks = (pl.k + tc::kBK - 1) / tc::kBK;
            g.tiles_m = tm2, g.tiles_n = tn2, g.bn = tc::kPairBN;
            g.total_tiles = tm2 * tn2 * pl.batch;
            g.stages = (budget - 8192u) / tc::kPairStageBytes;
            if (g.stages > 8) g.stages = 8;
            pl.smem_bytes = g.stages * tc::kPairStageBytes + 8192;
            pl.q_box_rows = g.q_major_mn ? 64 : 128;
            pl.workspace_bytes = pl.partials_bytes = pl.counters_bytes = 0;
            const uint64_t want = 2ull * g.total_tiles;
            pl.grid = (uint32_t) (want < 2ull * pairs ? want : 2ull * pairs);
        }
    }
    // D's lane index is c's row (or, transposed, its column)
    g.c_lane_stride = pl.swapped ? vc.col_stride : vc.row_stride;
    g.c_col_stride = pl.swapped ? vc.row_stride : vc.col_stride;
    g.c_batch_stride = vc.batch_stride;
    g.alpha = alpha, g.beta = beta;
    pl.use_tc = true;
    return STATUS_SUCCESS;
}

void matmul_plan_destroy(MatmulPlan &pl) {
    if (pl.counter_slot >= 0) counter_slot_release(pl.counter_slot);
    pl.counter_slot = -1;
}

static bool tc_pointers_ok(const MatmulPlan &pl, const void *a, const void *b) { return aligned16(a) && aligned16(b); }

infiniopStatus_t matmul_plan_run(MatmulPlan &pl, TcMapCache &cache, void *workspace, uint64_t workspace_size, void *c,
                                 const void *a, const void *b, cudaStream_t st) {
    if (pl.m == 0 || pl.n == 0 || pl.batch == 0) return STATUS_SUCCESS;
    const bool tc_path = pl.use_tc && tc_pointers_ok(pl, a, b) && kernel_choice(kFamilyMatmul) != 1 && pl.k > 0;
    if (tc_path) {
        tc::GemmParams g = pl.g;
        if (g.streamk) {
            if (workspace == nullptr || workspace_size < pl.workspace_bytes) return STATUS_INSUFFICIENT_WORKSPACE;
            unsigned char *w = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t) 255);
            g.partials = reinterpret_cast<float *>(w + pl.counters_bytes);
            uint32_t *pool = pl.counter_slot >= 0 ? counter_pool_address(pl.device_id) : nullptr;
            if (pool != nullptr) {
                // counters owned by the library: zero when the library is loaded, and every launch leaves them zero
                g.counters = pool + (size_t) pl.counter_slot * kSlotCounters;
            } else {
                g.counters = reinterpret_cast<uint32_t *>(w);
                if (cudaMemsetAsync(g.counters, 0, pl.counters_bytes, st) != cudaSuccess) return check_launch("matmul counters");
            }
        }
        const void *pp = pl.swapped ? b : a, *qp = pl.swapped ? a : b;
        {
            std::lock_guard<std::mutex> lock(cache.mu);
            if (!cache.valid || cache.p_ptr != pp || cache.q_ptr != qp) {
                if (!encode_operand(&cache.map_p, pp, pl.p, pl.p_box_rows, pl.bf16) ||
                    !encode_operand(&cache.map_q, qp, pl.q, pl.q_box_rows, pl.bf16)) {
                    fprintf(stderr, "infiniop[b200]: matmul: cuTensorMapEncodeTiled refused the operands\n");
                    return STATUS_EXECUTION_FAILED;
                }
                cache.p_ptr = pp, cache.q_ptr = qp, cache.valid = true;
            }
            g.c = reinterpret_cast<uint16_t *>(c);
            if (cudaFuncSetAttribute(tc::tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
                cudaSuccess) {
                return check_launch("matmul attribute");
            }
            if (pl.pair) {
                if (cudaFuncSetAttribute(tc::tc_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
                    cudaSuccess) {
                    return check_launch("matmul attribute");
                }
                launch_cluster_smem(tc::tc_gemm_pair_kernel, pl.grid, tc::kThreads, 2, pl.smem_bytes, st, cache.map_p,
                                    cache.map_q, g);
            } else {
                tc::tc_gemm_kernel<<<pl.grid, tc::kThreads, pl.smem_bytes, st>>>(cache.map_p, cache.map_q, g);
            }
        }
        return check_launch("matmul (tcgen05)");
    }
    if (pl.mode != tc::kEpiPlain) return STATUS_BAD_PARAM;// the fused epilogue exists on the tensor-core path only
    const dim3 grid((pl.n + kSimtTile - 1) / kSimtTile, (pl.m + kSimtTile - 1) / kSimtTile, pl.batch);
    if (grid.y > 65535 || grid.z > 65535) return STATUS_BAD_TENSOR_SHAPE;
    if (pl.f16) {
        auto *kernel = pl.bf16 ? matmul_simt_kernel<uint16_t, kBF16> : matmul_simt_kernel<uint16_t, kF16>;
        kernel<<<grid, 256, 0, st>>>(reinterpret_cast<uint16_t *>(c), reinterpret_cast<const uint16_t *>(a),
                                     reinterpret_cast<const uint16_t *>(b), pl.c, pl.a, pl.b, pl.m, pl.n, pl.k, pl.alpha,
                                     pl.beta);
    } else {
        matmul_simt_kernel<float, kF32><<<grid, 256, 0, st>>>(reinterpret_cast<float *>(c), reinterpret_cast<const float *>(a),
                                                      reinterpret_cast<const float *>(b), pl.c, pl.a, pl.b, pl.m, pl.n,
                                                      pl.k, pl.alpha, pl.beta);
    }
    return check_launch("matmul (cuda cores)");
}

unsigned long long tc_gemm_timeouts_read() {
    unsigned long long v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_tc_gemm_timeouts, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return ~0ull;
    }
    return v;
}

}// namespace b200

namespace {
struct MatmulDesc {
    Device device;
    MatmulPlan plan;
    TcMapCache cache;
};
}// namespace

INFINIOP_API infiniopStatus_t infiniopCreateMatmulDescriptor(infiniopHandle_t handle, infiniopMatmulDescriptor_t *desc_ptr,
                                                             infiniopTensorDescriptor_t c_desc, float alpha,
                                                             infiniopTensorDescriptor_t a_desc,
                                                             infiniopTensorDescriptor_t b_desc, float beta) {
    if (handle == nullptr || handle->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (desc_ptr == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    auto *d = new (std::nothrow) MatmulDesc;
    if (d == nullptr) return STATUS_MEMORY_NOT_ALLOCATED;
    d->device = DevNvGpu;
    d->plan.counter_slot = -1;
    const infiniopStatus_t s = matmul_plan_create(d->plan, reinterpret_cast<Handle *>(handle), c_desc, alpha, a_desc, b_desc,
                                                  beta, tc::kEpiPlain);
    if (s != STATUS_SUCCESS) {
        matmul_plan_destroy(d->plan);
        delete d;
        return s;
    }
    *desc_ptr = reinterpret_cast<infiniopMatmulDescriptor_t>(d);
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopGetMatmulWorkspaceSize(infiniopMatmulDescriptor_t desc, uint64_t *size) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (size == nullptr) return STATUS_BAD_PARAM;
    *size = reinterpret_cast<MatmulDesc *>(desc)->plan.workspace_bytes;
    return STATUS_SUCCESS;
}

INFINIOP_API infiniopStatus_t infiniopMatmul(infiniopMatmulDescriptor_t desc, void *workspace, uint64_t workspace_size,
                                             void *c, void const *a, void const *b, void *stream) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    if (c == nullptr || a == nullptr || b == nullptr) return STATUS_BAD_PARAM;
    auto *d = reinterpret_cast<MatmulDesc *>(desc);
    DeviceGuard guard(d->plan.device_id);
    return matmul_plan_run(d->plan, d->cache, workspace, workspace_size, c, a, b, reinterpret_cast<cudaStream_t>(stream));
}

INFINIOP_API infiniopStatus_t infiniopDestroyMatmulDescriptor(infiniopMatmulDescriptor_t desc) {
    if (desc == nullptr || desc->device != DevNvGpu) return STATUS_BAD_DEVICE;
    auto *d = reinterpret_cast<MatmulDesc *>(desc);
    matmul_plan_destroy(d->plan);
    delete d;
    return STATUS_SUCCESS;
}
