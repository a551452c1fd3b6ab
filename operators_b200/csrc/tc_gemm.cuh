// Tensor-core GEMM building blocks for sm_100a: TMA tile loads into 128-byte-swizzled shared memory,
// tcgen05.mma with the accumulator in tensor memory (TMEM), tcgen05.ld for the epilogue.
//
// The kernel computes D[Mp, Np] = sum_k P[Mp, k] * Q[Np, k] for fp16 operands with fp32 accumulation.
// P is the operand on the MMA's A side (its rows become TMEM lanes, 128 per tile), Q the one on the B side
// (its rows become TMEM columns, 16 .. 256 per tile).  Each operand may be K-major (k contiguous in memory) or
// MN-major (its row index contiguous); the host decides which of the caller's matrices plays P and which Q, so
// a product with few rows (decoding: a handful of tokens against a weight matrix) runs transposed with the
// weight matrix's output dimension on the 128 lanes and the tokens on 16 columns.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      one lane issues the TMA loads of a ring of kStages shared-memory stages (mbarrier full/empty)
//   warp 1      allocates TMEM; one lane issues tcgen05.mma per stage and commits stage and accumulator barriers
//   warps 2-5   epilogue: each reads its 32 TMEM lanes (tcgen05.ld), applies alpha / beta (or SwiGLU on the
//               gate and up halves) with the reference's truncating fp32 -> fp16 rule, and stores
// Two TMEM accumulator buffers let the epilogue of one tile overlap the main loop of the next.
//
// Work is a list of (tile, k-block range) items.  When the tiles alone cannot fill the GPU (decoding shapes),
// the k-blocks of all tiles are split evenly over the CTAs ("stream-K"): a CTA that owns only part of a tile's
// k range writes its fp32 partial tile to the workspace and counts itself on the tile; the CTA that arrives
// last adds the partials in CTA order (deterministic) and runs the epilogue.  Nobody waits for anybody.
//
// Every mbarrier wait is bounded (clock64 budget).  A role that runs out of time raises the CTA's abort flag
// and the device-wide counter g_tc_gemm_timeouts; all roles then leave their loops, the CTA waits (bounded)
// for its TMA copies in flight, frees its TMEM and returns.
#pragma once

#include "common.cuh"
#ifdef B200_TC_GEMM_KERNEL
#include "tc_ptx.cuh"
#endif

#include <cuda.h>
#include <type_traits>

namespace b200 {
namespace tc {

constexpr int kThreads = 192;
constexpr int kBM = 128;        // rows of P per tile = TMEM lanes
constexpr int kBK = 64;         // k per stage: 64 fp16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;      // k per tcgen05.mma (kind::f16)
constexpr uint32_t kPBytes = kBM * kBK * 2;// 16 KiB per stage for P

// kEpiSwiGLUCols: Q tiles hold [gate columns | matching up columns]; kEpiSwiGLULanes (transposed products): a tile
// is 128 features, their gate rows and their up rows of P feed two accumulators side by side in TMEM (p_tiles = 2),
// so a lane finds gate and up of its feature in its own columns.
enum EpilogueMode { kEpiPlain = 0, kEpiSwiGLUCols = 1, kEpiSwiGLULanes = 2 };

struct GemmParams {
    uint32_t mp, np, k;       // problem in MMA orientation
    uint32_t batch;
    uint32_t tiles_m, tiles_n;// per batch
    uint32_t p_tiles;         // 128-row tiles of P per k-block: 1, or 2 in lane-mode SwiGLU (gate rows, up rows)
    uint32_t kbs;             // 64-wide k-blocks per pipeline stage (1, 2 or 4)
    uint32_t kblocks;         // pipeline steps over k: ceil(k / (64 * kbs))
    uint32_t total_tiles;
    uint32_t bn;              // columns per tile (16 .. 256, multiple of 16)
    uint32_t q_boxes;         // TMA boxes per Q tile (1 for K-major, bn/64 for MN-major; doubled halves in SwiGLU mode)
    uint32_t q_box_bytes;
    uint32_t p_major_mn, q_major_mn;
    uint32_t bf16;            // operands and result are bf16 (an extension; the reference's matmul is fp16 / fp32)
    int32_t p_batch_mul, q_batch_mul;// 0 when the operand is broadcast over the batch
    uint32_t p_batch_div, q_batch_div;// operand batch = result batch / div (grouped heads share one operand)
    uint32_t stages;
    // stream-K
    uint32_t streamk;         // 0: whole tiles, round robin; 1: k-blocks split evenly
    uint32_t work_per_cta;
    float *partials;          // [grid][2][kBM * bn] fp32
    uint32_t *counters;       // [total_tiles], zero on entry
    // epilogue
    int mode;
    uint32_t half_offset;     // SwiGLU: distance (rows of Q, or of P in lane mode) between the gate half and the up half
    uint16_t *c;
    int64_t c_lane_stride, c_col_stride, c_batch_stride;// element strides of D's lane index / column index / batch
    float alpha, beta;
    // Causal structure of attention (rows = new tokens, row r sees columns j <= causal_total - causal_seq + r):
    // mode 1 (scores: D's columns are cached tokens) skips tiles that lie wholly behind the mask, nobody reads them;
    // mode 2 (values: k runs over cached tokens) stops a tile's k range where its last row's mask begins, the
    // probabilities behind it are exact zeros.  Not combined with the transposed orientation or stream-K.
    uint32_t causal_mode, causal_seq, causal_total;
};

// k-blocks (pipeline steps) tile (tm, tn) of `rows` x `cols` needs: all of them, none, or a causal prefix.
__device__ __forceinline__ uint32_t tile_kblocks(const GemmParams &p, uint32_t tm, uint32_t tn, uint32_t rows, uint32_t cols) {
    if (p.causal_mode == 0) return p.kblocks;
    uint32_t last_row = tm * rows + rows - 1;
    if (last_row > p.causal_seq - 1) last_row = p.causal_seq - 1;
    const uint32_t last_col = p.causal_total - p.causal_seq + last_row;// last visible column of the tile's last row
    if (p.causal_mode == 1) return tn * cols > last_col ? 0u : p.kblocks;
    const uint32_t per_step = kBK * p.kbs;
    const uint32_t need = (last_col + per_step) / per_step;// ceil((last_col + 1) / per_step)
    return need < p.kblocks ? need : p.kblocks;
}

// Everything below is device code and is compiled by the one translation unit that launches the kernel
// (it defines B200_TC_GEMM_KERNEL before including this header); other files only need the types above.
#ifdef B200_TC_GEMM_KERNEL

// ---------------------------------------------------------------- the kernel --
// Tile order: within a batch entry, bands of kRasterRows tile rows are walked column by column, so the CTAs that
// run at the same time share a few tile rows of P and a few tile columns of Q (about 16 + 9 tiles' worth of
// operands for 148 tiles in flight, instead of a whole operand), which keeps both in L2.
constexpr uint32_t kRasterRows = 16;
__device__ __forceinline__ void tile_coords(const GemmParams &p, uint32_t tile, uint32_t &b, uint32_t &tm, uint32_t &tn) {
    const uint32_t per_batch = p.tiles_m * p.tiles_n;
    b = tile / per_batch;
    const uint32_t r = tile - b * per_batch;
    const uint32_t band = r / (kRasterRows * p.tiles_n);
    const uint32_t in_band = r - band * (kRasterRows * p.tiles_n);
    const uint32_t rows_here = min(kRasterRows, p.tiles_m - band * kRasterRows);
    tn = in_band / rows_here;
    tm = band * kRasterRows + (in_band - tn * rows_here);
}

struct WorkItem {
    uint32_t tile, kb0, kb1;// k-block range [kb0, kb1)
};

// Item `it` of CTA `cta`; false when the CTA has no more items.
__device__ __forceinline__ bool work_item(const GemmParams &p, uint32_t cta, uint32_t grid, uint32_t it, WorkItem &w) {
    if (!p.streamk) {
        const uint64_t t = (uint64_t) cta + (uint64_t) it * grid;
        if (t >= p.total_tiles) return false;
        w.tile = (uint32_t) t, w.kb0 = 0, w.kb1 = p.kblocks;
        if (p.causal_mode != 0) {
            uint32_t b, tm, tn;
            tile_coords(p, w.tile, b, tm, tn);
            w.kb1 = tile_kblocks(p, tm, tn, kBM, p.bn);// 0: the tile lies behind the causal mask and is skipped
        }
        return true;
    }
    const uint64_t total = (uint64_t) p.total_tiles * p.kblocks;
    const uint64_t begin = (uint64_t) cta * p.work_per_cta;
    uint64_t end = begin + p.work_per_cta;
    if (end > total) end = total;
    if (begin >= end) return false;
    const uint32_t first_tile = (uint32_t) (begin / p.kblocks);
    const uint32_t tile = first_tile + it;
    const uint64_t t0 = (uint64_t) tile * p.kblocks;
    if (t0 >= end) return false;
    w.tile = tile;
    w.kb0 = t0 < begin ? (uint32_t) (begin - t0) : 0u;
    w.kb1 = t0 + p.kblocks > end ? (uint32_t) (end - t0) : p.kblocks;
    return true;
}

// The 16-bit storage type of D and of the intermediate the SwiGLU epilogue rounds through: fp16 with the reference's
// truncating rule, or bf16 truncated likewise.
// (the type is decided once per 16 columns, so that the loops over the columns carry no branch)
template<bool BF16>
__device__ __forceinline__ uint16_t to_store16(float v) {
    return BF16 ? f32_to_bf16_trunc(v) : f32_to_f16_ref(v);
}
template<bool BF16>
__device__ __forceinline__ float load_store16(uint16_t h) {
    return BF16 ? __uint_as_float((uint32_t) h << 16) : f16_to_f32(h);
}
// gate[j] = up[j] * silu(gate[j]) on values rounded through the storage type, as the reference stores x * w12 before
// SwiGLU reads it back
template<bool BF16>
__device__ __forceinline__ void swiglu16_t(float *gate, const float *up) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float g = load_store16<BF16>(to_store16<BF16>(gate[j])), u = load_store16<BF16>(to_store16<BF16>(up[j]));
        gate[j] = __fmul_rn(u, silu_f32(g));
    }
}
__device__ __forceinline__ void swiglu16(const GemmParams &p, float *gate, const float *up) {
    if (p.bf16) swiglu16_t<true>(gate, up);
    else swiglu16_t<false>(gate, up);
}

// Final values of 16 consecutive columns of one lane, written to D.
__device__ __forceinline__ void store_cols16(const GemmParams &p, const float *acc, uint32_t row, uint32_t col0,
                                             uint32_t batch, uint32_t mp, uint32_t np, float alpha, float beta) {
    if (row >= mp) return;
    uint16_t *base = p.c + (int64_t) batch * p.c_batch_stride + (int64_t) row * p.c_lane_stride;
    uint16_t out[16];
    auto convert = [&](auto bf16) {
        constexpr bool kBf16 = decltype(bf16)::value;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float v = __fmul_rn(alpha, acc[j]);
            if (beta != 0.f && col0 + j < np) {
                v = __fadd_rn(__fmul_rn(beta, load_store16<kBf16>(base[(int64_t) (col0 + j) * p.c_col_stride])), v);
            }
            out[j] = to_store16<kBf16>(v);
        }
    };
    if (p.bf16) convert(std::true_type{});
    else convert(std::false_type{});
    if (p.c_col_stride == 1 && col0 + 16 <= np && ((reinterpret_cast<uintptr_t>(base + col0) & 15u) == 0)) {
        uint4 *dst = reinterpret_cast<uint4 *>(base + col0);
        const uint4 *src = reinterpret_cast<const uint4 *>(out);
        dst[0] = src[0];
        dst[1] = src[1];
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (col0 + j < np) base[(int64_t) (col0 + j) * p.c_col_stride] = out[j];
        }
    }
}

// The epilogue of one tile for one lane: `load16(c, v)` delivers the 16 accumulator columns that start at
// column c of the tile (from TMEM, or from the summed stream-K partials).
template<typename Load16>
__device__ __forceinline__ void finish_tile(const GemmParams &p, Load16 load16, uint32_t lane_row, uint32_t tm,
                                            uint32_t tn, uint32_t b) {
    if (p.mode == kEpiSwiGLUCols) {
        const uint32_t half = p.bn / 2, row = tm * kBM + lane_row;
        for (uint32_t c0 = 0; c0 < half; c0 += 16) {
            float gate[16], up[16];
            load16(c0, gate);
            load16(half + c0, up);
            swiglu16(p, gate, up);
            store_cols16(p, gate, row, tn * half + c0, b, p.mp, p.half_offset, 1.f, 0.f);
        }
    } else if (p.mode == kEpiSwiGLULanes) {
        const uint32_t feature = tm * kBM + lane_row;// columns [0, bn): gate, [bn, 2 bn): up, both of this feature
        for (uint32_t c0 = 0; c0 < p.bn; c0 += 16) {
            float gate[16], up[16];
            load16(c0, gate);
            load16(p.bn + c0, up);
            swiglu16(p, gate, up);
            store_cols16(p, gate, feature, tn * p.bn + c0, b, p.half_offset, p.np, 1.f, 0.f);// result rows = features
        }
    } else {
        const uint32_t row = tm * kBM + lane_row;
        for (uint32_t c0 = 0; c0 < p.bn; c0 += 16) {
            float acc[16];
            load16(c0, acc);
            store_cols16(p, acc, row, tn * p.bn + c0, b, p.mp, p.np, p.alpha, p.beta);
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1)
    tc_gemm_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                   const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // carve: stages of (P tile, Q tile), 1024-byte aligned; then barriers and flags
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    const uint32_t q_bytes = p.q_boxes * p.q_box_bytes;
    const uint32_t p_bytes = p.p_tiles * kPBytes;
    const uint32_t sub_bytes = p_bytes + ((q_bytes + 1023u) & ~1023u);// one 64-wide k-block of P and Q
    const uint32_t stage_bytes = p.kbs * sub_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t) p.stages * stage_bytes);
    uint64_t *full = bars, *empty = bars + p.stages, *acc_full = bars + 2 * p.stages, *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    uint32_t *last_flag = tmem_slot + 2;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t acc_cols = p.p_tiles * p.bn;                   // fp32 columns per accumulator buffer
    uint32_t tmem_cols = 32;
    while (tmem_cols < 2 * acc_cols) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_q);
    }
    // The producer does not need the TMEM address: warp 0 only announces that the barriers exist (bar.arrive) and
    // starts loading, while warp 1 allocates TMEM and the other warps wait for both.
    uint32_t tmem_base = 0;
    if (warp == 0) {
        __syncwarp();
        asm volatile("bar.arrive 3, %0;" ::"n"(kThreads) : "memory");
    } else {
        if (warp == 1) {
            tmem_alloc(tmem_slot, tmem_cols);
            tmem_relinquish();
        }
        tc_fence_before();
        asm volatile("bar.sync 3, %0;" ::"n"(kThreads) : "memory");
        tc_fence_after();
        tmem_base = *tmem_slot;
    }

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            WorkItem w;
            bool ok = true;
            for (uint32_t it = 0; ok && work_item(p, blockIdx.x, gridDim.x, it, w); ++it) {
                uint32_t b, tm, tn;
                tile_coords(p, w.tile, b, tm, tn);
                for (uint32_t kb = w.kb0; kb < w.kb1; ++kb) {// no pass for a tile behind the causal mask
                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    unsigned char *sbase = smem + (size_t) stage * stage_bytes;
                    mbar_expect_tx(&full[stage], p.kbs * (p_bytes + q_bytes));
                    const int32_t pb = (int32_t) (b / p.p_batch_div) * p.p_batch_mul, qb = (int32_t) (b / p.q_batch_div) * p.q_batch_mul;
                    // P first: the boxes of one step continue each other's rows in memory, so their requests reach
                    // the memory system together (256 or 512 contiguous bytes per row instead of 128)
                    for (uint32_t sub = 0; sub < p.kbs; ++sub) {
                        unsigned char *sp = sbase + (size_t) sub * sub_bytes;
                        const int32_t k0 = (int32_t) ((kb * p.kbs + sub) * kBK);
                        for (uint32_t t = 0; t < p.p_tiles; ++t) {// lane-mode SwiGLU: the gate rows, then the up rows
                            unsigned char *dst = sp + (size_t) t * kPBytes;
                            const int32_t r0 = (int32_t) (tm * kBM + t * p.half_offset);
                            if (!p.p_major_mn) {
                                tma_load_3d(dst, &map_p, &full[stage], k0, r0, pb);
                            } else {
                                tma_load_3d(dst, &map_p, &full[stage], r0, k0, pb);
                                tma_load_3d(dst + kPBytes / 2, &map_p, &full[stage], r0 + 64, k0, pb);
                            }
                        }
                    }
                    for (uint32_t sub = 0; sub < p.kbs; ++sub) {
                        unsigned char *sq = sbase + (size_t) sub * sub_bytes + p_bytes;
                        const int32_t k0 = (int32_t) ((kb * p.kbs + sub) * kBK);
                        if (p.mode == kEpiSwiGLUCols) {
                            // Q tile = gate columns [tn * bn/2, +bn/2) followed by the matching up columns
                            const uint32_t half = p.bn / 2, boxes_half = p.q_boxes / 2;
                            for (uint32_t h = 0; h < 2; ++h) {
                                const int32_t r0 = (int32_t) (tn * half + h * p.half_offset);
                                for (uint32_t x = 0; x < boxes_half; ++x) {
                                    unsigned char *dst = sq + (size_t) (h * boxes_half + x) * p.q_box_bytes;
                                    if (!p.q_major_mn) tma_load_3d(dst, &map_q, &full[stage], k0, r0, qb);
                                    else tma_load_3d(dst, &map_q, &full[stage], r0 + (int32_t) (x * 64), k0, qb);
                                }
                            }
                        } else if (!p.q_major_mn) {
                            tma_load_3d(sq, &map_q, &full[stage], k0, (int32_t) (tn * p.bn), qb);
                        } else {
                            for (uint32_t x = 0; x < p.q_boxes; ++x) {
                                tma_load_3d(sq + (size_t) x * p.q_box_bytes, &map_q, &full[stage],
                                            (int32_t) (tn * p.bn + x * 64), k0, qb);
                            }
                        }
                    }
                    if (++stage == p.stages) stage = 0, phase ^= 1u;
                }
            }
        }
        __syncwarp();// the other lanes wait here, so the warp reaches the closing barrier converged
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc(kBM, p.bn, p.p_major_mn, p.q_major_mn, p.bf16);
            uint32_t stage = 0, phase = 0, acc_it = 0;
            WorkItem w;
            bool ok = true;
            for (uint32_t it = 0; ok && work_item(p, blockIdx.x, gridDim.x, it, w); ++it) {
                if (w.kb1 <= w.kb0) continue;// a tile behind the causal mask: no accumulator, no epilogue
                const uint32_t buf = acc_it & 1u;
                if (!mbar_wait(&acc_empty[buf], ((acc_it >> 1) & 1u) ^ 1u, abort_flag)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * acc_cols;
                for (uint32_t kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    for (uint32_t sub = 0; sub < p.kbs; ++sub) {
                        const uint32_t sp0 = smem_u32(smem + (size_t) stage * stage_bytes + (size_t) sub * sub_bytes);
                        const uint32_t sq = sp0 + p_bytes;
                        for (uint32_t t = 0; t < p.p_tiles; ++t) {
                            const uint32_t sp = sp0 + t * kPBytes;
#pragma unroll
                            for (uint32_t j = 0; j < kBK / kUmmaK; ++j) {
                                // K-major: 16 k = 32 bytes further along the swizzled 128-byte rows, 8-row groups 1024
                                // bytes apart.  MN-major: 16 k = two 8-row groups of 1024 bytes; 64-row atoms one TMA
                                // box apart.
                                const uint64_t da = p.p_major_mn ? make_smem_desc(sp + j * 2048u, kPBytes / 2, 1024)
                                                                 : make_smem_desc(sp + j * 32u, 16, 1024);
                                const uint64_t db = p.q_major_mn ? make_smem_desc(sq + j * 2048u, p.q_box_bytes, 1024)
                                                                 : make_smem_desc(sq + j * 32u, 16, 1024);
                                umma_f16(d_tmem + t * p.bn, da, db, idesc, (kb > w.kb0 || sub > 0 || j > 0) ? 1u : 0u);
                            }
                        }
                    }
                    umma_commit(&empty[stage]);// the stage may be refilled once these MMAs have read it
                    if (++stage == p.stages) stage = 0, phase ^= 1u;
                }
                if (ok) umma_commit(&acc_full[buf]);
                ++acc_it;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const uint32_t quarter = warp & 3u;// TMEM lanes 32 * quarter .. + 31 belong to this warp
        const uint32_t epi_tid = (warp - 2) * 32 + lane;
        uint32_t acc_it = 0;
        WorkItem w;
        for (uint32_t it = 0; work_item(p, blockIdx.x, gridDim.x, it, w); ++it) {
            if (w.kb1 <= w.kb0) continue;
            const uint32_t buf = acc_it & 1u;
            uint32_t b, tm, tn;
            tile_coords(p, w.tile, b, tm, tn);
            if (!mbar_wait(&acc_full[buf], (acc_it >> 1) & 1u, abort_flag)) break;
            tc_fence_after();
            const uint32_t lane_row = quarter * 32 + lane;
            // does this lane hold a row of the matrix (lane mode: a feature below the intermediate size)?
            const bool row_valid = tm * kBM + lane_row < p.mp;
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + buf * acc_cols;
            const bool partial = p.streamk && !(w.kb0 == 0 && w.kb1 == p.kblocks);
            if (!partial) {
                finish_tile(p, [&](uint32_t c, float *v) { tmem_ld16(taddr + c, v); }, lane_row, tm, tn, b);
                tc_fence_before();
                mbar_arrive(&acc_empty[buf]);
            } else {
                // part of a tile's k range: park the fp32 partial, count this CTA on the tile, and let the CTA
                // that arrives last add all parts in CTA order
                const uint32_t slot = w.kb0 == 0 ? 1u : 0u;// a part that starts mid-tile opens the CTA's range (slot 0)
                float *mine = p.partials + ((size_t) blockIdx.x * 2 + slot) * (size_t) (kBM * acc_cols);
                for (uint32_t c0 = 0; c0 < acc_cols; c0 += 16) {
                    float acc[16];
                    tmem_ld16(taddr + c0, acc);// all lanes of the warp take part in the load
                    if (row_valid) {           // rows beyond the matrix are never read back
                        float4 *dst = reinterpret_cast<float4 *>(mine + (size_t) lane_row * acc_cols + c0);
#pragma unroll
                        for (int j = 0; j < 4; ++j) __stcg(dst + j, make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
                    }
                }
                tc_fence_before();
                mbar_arrive(&acc_empty[buf]);
                asm volatile("bar.sync 1, 128;" ::: "memory");// the four epilogue warps: all parts are written
                // CTAs whose range meets this tile: first .. last
                const uint64_t t0 = (uint64_t) w.tile * p.kblocks;
                const uint32_t first = (uint32_t) (t0 / p.work_per_cta);
                const uint32_t last = (uint32_t) ((t0 + p.kblocks - 1) / p.work_per_cta);
                if (epi_tid == 0) {
                    __threadfence();// release: the barrier above made the other threads' stores this thread's to publish
                    const uint32_t seen = atomicAdd(&p.counters[w.tile], 1u);
                    *last_flag = seen == last - first ? 1u : 0u;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool is_last = *last_flag != 0;// rewritten only behind the next part's first barrier
                if (is_last) {
                    __threadfence();
                    if (epi_tid == 0) p.counters[w.tile] = 0;// ready for the next launch
                    finish_tile(
                        p,
                        [&](uint32_t c, float *acc) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
                            if (!row_valid) return;
                            for (uint32_t cta = first; cta <= last; ++cta) {
                                // CTA `cta`'s part of this tile starts mid-tile exactly when its range starts inside the tile
                                const uint64_t cb = (uint64_t) cta * p.work_per_cta;
                                const uint32_t s = cb > t0 ? 0u : 1u;
                                const float *src = p.partials + ((size_t) cta * 2 + s) * (size_t) (kBM * acc_cols) +
                                                   (size_t) lane_row * acc_cols + c;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float4 v = __ldcg(reinterpret_cast<const float4 *>(src) + j);
                                    acc[4 * j] += v.x, acc[4 * j + 1] += v.y, acc[4 * j + 2] += v.z, acc[4 * j + 3] += v.w;
                                }
                            }
                        },
                        lane_row, tm, tn, b);
                }
            }
            ++acc_it;
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // let TMA copies that are still in flight land before the shared memory is given back
        for (uint32_t s = 0; s < p.stages; ++s) {
            const long long t0 = clock64();
            while (!mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1) && clock64() - t0 < 2000000ll) {}
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2) --
// Large products: a cluster of two CTAs owns a 256 x 256 tile.  Each CTA loads its 128 rows of P and its 128
// rows of Q per stage (32 KB instead of the 48 KB a lone CTA needs for 128 x 256), the leader CTA issues
// tcgen05.mma.cta_group::2 (M = 256 over both CTAs, each reading the other's half of Q from its shared memory),
// and each CTA finds its 128 rows of the accumulator in its own tensor memory.  One CTA alone spends the shared
// memory port twice over (TMA writes plus operand reads of A and all of B: 192 bytes per cycle at the full MMA
// rate against a 128-byte port); the pair needs 128.  Barriers: the peer's TMA loads complete on the LEADER's
// full barrier (cta_group::2 form of the copy), the leader's commits are multicast to both CTAs' empty and
// accumulator barriers, the peer's epilogue arrives on the leader's accumulator-empty barrier remotely.  The loads
// themselves carry no multicast.  Plain and column-mode SwiGLU epilogues; no stream-K.
// TMA load whose mbarrier may live in the peer CTA of the pair (address in the cluster window).
__device__ __forceinline__ void tma_load_3d_pair(void *smem_dst, const CUtensorMap *map, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y, int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// one arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair, once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask)
                 : "memory");
}

constexpr uint32_t kPairBN = 256;
constexpr uint32_t kPairStageBytes = 2 * kPBytes;// 128 x 64 of P and 128 x 64 of Q per CTA

// Tile `it` of pair `pair` (round robin over the pairs); tiles are 256 x 256.
__device__ __forceinline__ bool pair_tile(const GemmParams &p, uint32_t pair, uint32_t pairs, uint32_t it, uint32_t &tile) {
    const uint64_t t = (uint64_t) pair + (uint64_t) it * pairs;
    if (t >= p.total_tiles) return false;
    tile = (uint32_t) t;
    return true;
}

__global__ void __launch_bounds__(kThreads, 1)
    tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                        const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t) p.stages * kPairStageBytes);
    uint64_t *full = bars, *empty = bars + p.stages, *acc_full = bars + 2 * p.stages, *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();// 0 = leader
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    constexpr uint32_t kTmemCols = 512;  // two accumulators of 256 fp32 columns

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1); // the leader's arrive.expect_tx; bytes from both CTAs (used in the leader only)
            mbar_init(&empty[s], 1);// one multicast commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);   // one multicast commit
            mbar_init(&acc_empty[b], 256);// the epilogue threads of both CTAs (used in the leader only)
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_q);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();// both CTAs' barriers are initialised before anybody signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one lane in each CTA)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, tile;
            bool ok = true;
            for (uint32_t it = 0; ok && pair_tile(p, pair, pairs, it, tile); ++it) {
                uint32_t b, tm, tn;
                tile_coords(p, tile, b, tm, tn);
                const int32_t pb = (int32_t) (b / p.p_batch_div) * p.p_batch_mul, qb = (int32_t) (b / p.q_batch_div) * p.q_batch_mul;
                const int32_t prow = (int32_t) (tm * 256 + rank * 128);
                // rows of Q this CTA holds: its half of the 256 columns, or (SwiGLU) the gate half in the leader and
                // the matching up half in the peer
                const int32_t qrow = p.mode == kEpiSwiGLUCols ? (int32_t) (tn * 128 + rank * p.half_offset)
                                                              : (int32_t) (tn * 256 + rank * 128);
                const uint32_t kbs_here = tile_kblocks(p, tm, tn, 256, kPairBN);// 0: behind the causal mask
                for (uint32_t kb = 0; kb < kbs_here; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    unsigned char *sp = smem + (size_t) stage * kPairStageBytes, *sq = sp + kPBytes;
                    const uint32_t full_leader = mapa_u32(smem_u32(&full[stage]), 0);
                    if (rank == 0) mbar_expect_tx(&full[stage], 2 * kPairStageBytes);
                    const int32_t k0 = (int32_t) (kb * kBK);
                    if (!p.p_major_mn) {
                        tma_load_3d_pair(sp, &map_p, full_leader, k0, prow, pb);
                    } else {
                        tma_load_3d_pair(sp, &map_p, full_leader, prow, k0, pb);
                        tma_load_3d_pair(sp + kPBytes / 2, &map_p, full_leader, prow + 64, k0, pb);
                    }
                    if (!p.q_major_mn) {
                        tma_load_3d_pair(sq, &map_q, full_leader, k0, qrow, qb);
                    } else {
                        tma_load_3d_pair(sq, &map_q, full_leader, qrow, k0, qb);
                        tma_load_3d_pair(sq + kPBytes / 2, &map_q, full_leader, qrow + 64, k0, qb);
                    }
                    if (++stage == p.stages) stage = 0, phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc(256, kPairBN, p.p_major_mn, p.q_major_mn, p.bf16);
            uint32_t stage = 0, phase = 0, acc_it = 0, tile;
            bool ok = true;
            for (uint32_t it = 0; ok && pair_tile(p, pair, pairs, it, tile); ++it) {
                uint32_t b, tm, tn;
                tile_coords(p, tile, b, tm, tn);
                const uint32_t kbs_here = tile_kblocks(p, tm, tn, 256, kPairBN);
                if (kbs_here == 0) continue;
                const uint32_t buf = acc_it & 1u;
                if (!mbar_wait(&acc_empty[buf], ((acc_it >> 1) & 1u) ^ 1u, abort_flag)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * kPairBN;
                for (uint32_t kb = 0; kb < kbs_here; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sp = smem_u32(smem + (size_t) stage * kPairStageBytes), sq = sp + kPBytes;
#pragma unroll
                    for (uint32_t j = 0; j < kBK / kUmmaK; ++j) {
                        const uint64_t da = p.p_major_mn ? make_smem_desc(sp + j * 2048u, kPBytes / 2, 1024)
                                                         : make_smem_desc(sp + j * 32u, 16, 1024);
                        const uint64_t db = p.q_major_mn ? make_smem_desc(sq + j * 2048u, kPBytes / 2, 1024)
                                                         : make_smem_desc(sq + j * 32u, 16, 1024);
                        umma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&empty[stage]);
                    if (++stage == p.stages) stage = 0, phase ^= 1u;
                }
                if (ok) umma_commit_pair(&acc_full[buf]);
                ++acc_it;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
        const uint32_t quarter = warp & 3u;
        uint32_t acc_it = 0, tile;
        for (uint32_t it = 0; pair_tile(p, pair, pairs, it, tile); ++it) {
            uint32_t b, tm, tn;
            tile_coords(p, tile, b, tm, tn);
            if (tile_kblocks(p, tm, tn, 256, kPairBN) == 0) continue;
            const uint32_t buf = acc_it & 1u;
            if (!mbar_wait(&acc_full[buf], (acc_it >> 1) & 1u, abort_flag)) break;
            tc_fence_after();
            const uint32_t lane_row = quarter * 32 + lane;
            const uint32_t row = tm * 256 + rank * 128 + lane_row;
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + buf * kPairBN;
            if (p.mode == kEpiSwiGLUCols) {
                for (uint32_t c0 = 0; c0 < 128; c0 += 16) {
                    float gate[16], up[16];
                    tmem_ld16(taddr + c0, gate);
                    tmem_ld16(taddr + 128 + c0, up);
                    swiglu16(p, gate, up);
                    store_cols16(p, gate, row, tn * 128 + c0, b, p.mp, p.half_offset, 1.f, 0.f);
                }
            } else {
                for (uint32_t c0 = 0; c0 < kPairBN; c0 += 16) {
                    float acc[16];
                    tmem_ld16(taddr + c0, acc);
                    store_cols16(p, acc, row, tn * kPairBN + c0, b, p.mp, p.np, p.alpha, p.beta);
                }
            }
            tc_fence_before();
            mbar_arrive_remote(mapa_u32(smem_u32(&acc_empty[buf]), 0));
            ++acc_it;
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000ll) {}// copies in flight towards either CTA land (about 2 ms)
    }
    cluster_sync_all();// nobody leaves while the other CTA may still signal its barriers or read its shared memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

#endif// B200_TC_GEMM_KERNEL

}// namespace tc
}// namespace b200
