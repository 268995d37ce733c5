// Tensor-core linear kernel for prefill and large batches (M > 16), sm_100a:
//   out[M,N] = x[M,K] . W[N,K]^T, fp16 operands, fp32 accumulation in tensor memory.
//
// Stands in for the reference's M > 1 path, a CLBlast Gemm<cl_half> call
// (src/models/lfm2-5-350m/src/utils.cpp:1334-1345: RowMajor, A no-trans, B trans,
// lda = ldb = K, ldc = N, alpha 1, beta 0), and for its token-by-token loop over
// quantised weights (src/models/lfm2-5-350m/src/model.cpp:243-251).
//
// Persistent blocks (one per SM) walk 128 (weight rows) x BN (tokens, <= 256) output tiles,
// each over all of K, with two accumulators in tensor memory so that the epilogue of one
// tile overlaps the MMAs of the next:
//   * warp 0, one lane: TMA producer.  Per 64-wide K block it issues two tiled tensor
//     copies (cp.async.bulk.tensor.2d, 128-byte swizzle): 128 weight rows and BN
//     activation rows, both K-major, completing on the stage's "full" mbarrier.
//   * warp 1, one lane: issues tcgen05.mma (cta_group::1, kind::f16, M128 x N(BN) x K16,
//     four per K block) on shared-memory descriptors; the accumulator lives in tensor
//     memory (128 lanes x BN fp32 columns).  tcgen05.commit hands each stage back through
//     its "empty" mbarrier and signals the epilogue at the end.
//   * warps 2-5: epilogue.  Warp w reads lanes 32 (w % 4) .. +31 of the accumulator with
//     tcgen05.ld (lane = weight row, column = token), applies the per-row int8 scale or
//     the in-place residual, converts to fp16 and stores; for a fixed token the 32 lanes
//     of a warp write 32 consecutive outputs.
// Blocks that share a weight tile (different token tiles) are adjacent in launch order, so
// the tile is fetched from HBM once and re-read from L2.
//
// int8 / Q4 weights are streamed packed, once: four more warps expand each stage into the fp16
// operand inside shared memory (int8 codes are exact in fp16 and the per-row scale is applied in
// the epilogue, after the full-K sum, like the GEMV; Q4 becomes code x block-scale rounded to fp16).
#include <cuda.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nnb {
namespace {

constexpr int BM = 128;       // weight rows per tile (UMMA M)
constexpr int BK = 64;        // K elements per stage = one 128-byte swizzle span of fp16
constexpr int EPI_WARPS = 4;
// quantised weights only: warps that turn the packed stage into the fp16 operand, in groups of four
// that take K blocks in turn (int8: two groups, Q4, whose expansion is heavier: four)
__host__ __device__ constexpr int dq_warps(int wfmt) { return wfmt == FMT_Q4 ? 16 : wfmt == FMT_INT8 ? 8 : 0; }
constexpr int GEMM_THREADS = (2 + EPI_WARPS) * 32;            // producer warp, MMA warp, four epilogue warps
__host__ __device__ constexpr int gemm_threads(int wfmt) {    // ... plus the expanding warps and the packed-weight producer
    return wfmt == FMT_FP16 ? GEMM_THREADS : GEMM_THREADS + dq_warps(wfmt) * 32 + 32;
}
constexpr int A_BYTES = BM * BK * 2;  // 16 KB
constexpr int OUT_ROWS = 128;         // tokens per output slab (staging buffer: OUT_ROWS x 128 fp16 = 32 KB)

struct GemmK {
    alignas(64) CUtensorMap tm_w;  // fp16: [N][K] half, box 64 x 128; int8: [N][K] bytes, Q4: [N][K/2] bytes, box 128 B x 128
                                   // (all with the 128-byte swizzle)
    const uint16_t* q4_scale;      // Q4: [N][K/32] fp16 block scales (read by the dequantising warps)
    alignas(64) CUtensorMap tm_x;  // [M][K] fp16, box 64 x BN
    alignas(64) CUtensorMap tm_out;  // [M][ld_out] fp16, box 128 x BN (dense), when tma_store
    int tma_store;                   // plain-store epilogue through shared memory and one tensor store per tile
    uint16_t* out;                 // [M][ld_out]
    const uint16_t* row_scale;     // int8 weights: fp16 scale per weight row, else null
    int M, N, K, ld_out;
    int bn;        // tokens per tile (multiple of 16, <= 256)
    int ntok;      // token tiles
    int stages;
    int raw_stages;  // packed weights: depth of their own, deeper ring (covers the HBM latency)
    int tmem_cols; // power of two >= bn
    int epi;       // EPI_STORE or EPI_RESIDUAL
    int* status;
    uint16_t* peer_out[7];  // the same output block in the other ranks' gather buffers
    int npeer;
    GatherSignal sig;       // completion signal of the gather (world == 0: none)
};

// ---- tcgen05 wrappers -------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- tensor store (shared -> global) ------------------------------------------------------
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src), "r"(x), "r"(y)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand in 128-byte-swizzled rows of 128 bytes:
// start address >> 4, stride between 8-row groups = 1024 bytes, descriptor version 1,
// layout type 2 (128-byte swizzle).  The leading-dimension offset is not used by this layout.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                       // leading byte offset field (unused for swizzled K-major)
    d |= (uint64_t)((1024 >> 4) & 0x3FFF) << 32;  // stride byte offset
    d |= (uint64_t)1 << 46;                       // version
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}

// The same descriptor from its halves: the high word never changes, the low word is the 16-byte address (14 bits) plus
// the constant leading-offset field, so a K step of 32 bytes inside a swizzle span is "+ 2" on the low word.
constexpr uint32_t DESC_HI = (uint32_t)((1024 >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t saddr) { return ((saddr >> 4) & 0x3FFFu) | (1u << 16); }
__device__ __forceinline__ uint64_t desc_of(uint32_t lo) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(DESC_HI));
    return d;
}

// Instruction descriptor: fp32 accumulate, fp16 x fp16, both operands K-major, M = 128, N = bn.
__device__ __forceinline__ uint32_t instr_desc_f16(int bn) {
    uint32_t d = 0;
    d |= 1u << 4;                       // c_format = F32
    d |= 0u << 7;                       // a_format = F16
    d |= 0u << 10;                      // b_format = F16
    d |= (uint32_t)(bn >> 3) << 17;     // n_dim
    d |= (uint32_t)(BM >> 4) << 24;     // m_dim
    return d;
}

// WFMT = FMT_FP16: the weight operand is loaded by TMA as it is.  FMT_INT8 / FMT_Q4: TMA brings the
// packed rows of a stage, four more warps expand them to fp16 straight into the MMA's swizzled
// operand layout (int8 codes are exact in fp16 and the row scale is applied in the epilogue; a Q4
// weight becomes fp16(code * block scale)), so a quantised weight is read from HBM once, packed.
template <int WFMT>
__global__ void __launch_bounds__(gemm_threads(WFMT)) linear_gemm_tc_kernel(const __grid_constant__ GemmK g) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int DQ_WARPS = dq_warps(WFMT), NGRP = DQ_WARPS >= 4 ? DQ_WARPS / 4 : 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t s_base = smem_u32(smem);
    // Scalars are read from the parameter block once: its address is taken (tensor maps), so a
    // field read after a store would be a fresh load each time, and the epilogue stores a lot.
    const int gM = g.M, gN = g.N, g_ld = g.ld_out, g_bn = g.bn, g_ntok = g.ntok, g_stages = g.stages, g_cols = g.tmem_cols;
    const int g_epi = g.epi, g_npeer = g.npeer, g_tma_store = g.tma_store;
    uint16_t* const g_out = g.out;
    const uint16_t* const g_rs = g.row_scale;
    int* const g_status = g.status;
    uint16_t* g_peer[7];
#pragma unroll
    for (int p = 0; p < 7; ++p) g_peer[p] = p < g_npeer ? g.peer_out[p] : nullptr;
    // header: full[S] @0, empty[S] @64, acc_full[2] @128, acc_empty[2] @144, tensor-memory address @160,
    // residual-tile barrier @176
    const uint32_t full0 = s_base, empty0 = s_base + 64, acc_full0 = s_base + 128, acc_empty0 = s_base + 144, tmem_slot = s_base + 160;
    const uint32_t res_bar = s_base + 176, raw_full0 = s_base + 192, raw_empty0 = s_base + 256;  // up to 8 packed stages
    const uint32_t ring = (s_base + 1024u + 1023u) & ~1023u;
    const int b_bytes = g_bn * BK * 2;
    // Packed weights arrive in spans of 128 bytes per row (int8: two K blocks, Q4: four), so that the
    // HBM reads are 128-byte pieces rather than 32- or 64-byte ones; 128-byte swizzle, like the operands.
    constexpr int RAW_SPAN = WFMT == FMT_INT8 ? 2 : 4;       // K blocks per packed stage
    constexpr int RAW_BYTES = WFMT == FMT_FP16 ? 0 : BM * 128;
    const int stage_bytes = A_BYTES + ((b_bytes + 1023) / 1024) * 1024;
    const int g_raw_stages = g.raw_stages;
    const int nkb = (g.K + BK - 1) / BK;
    const uint32_t raw_ring = ring + (uint32_t)(g_stages * stage_bytes);        // packed weight stages
    const uint32_t out_stage = raw_ring + (uint32_t)(g_raw_stages * RAW_BYTES);  // fp16 staging of one output slab
    const int ntiles = ((gN + BM - 1) / BM) * g_ntok;

    if (tid == 0) {
        for (int s = 0; s < g_stages; ++s) {
            mbar_init(full0 + s * 8, WFMT == FMT_FP16 ? 1 : 1 + 4);  // operands ready: TMA bytes (+ one group of four expanding warps)
            mbar_init(empty0 + s * 8, 1);
        }
        for (int r = 0; r < g_raw_stages; ++r) {
            mbar_init(raw_full0 + r * 8, 1);
            mbar_init(raw_empty0 + r * 8, DQ_WARPS);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full0 + a * 8, 1);
            mbar_init(acc_empty0 + a * 8, EPI_WARPS);
        }
        mbar_init(res_bar, 1);
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_slot, (uint32_t)(2 * g_cols));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem + 160);

    if (warp == 0) {
        // ---- TMA producer: one lane walks (tile, K block) and keeps the ring full ----
        if (lane == 0) {
            const uint64_t policy = l2_policy_evict_normal();
            int it = 0, s = 0;
            uint32_t ph = 0;   // parity of the ring pass (it / g_stages) & 1, kept without divisions
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int wt = tile / g_ntok, tt = tile - wt * g_ntok;
                for (int kb = 0; kb < nkb; ++kb, ++it, s = (s + 1 == g_stages ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
                    if (it >= g_stages && !mbar_wait_bounded(empty0 + s * 8, ph ^ 1u)) {
                        *reinterpret_cast<volatile int*>(g_status) = 3;
                        ok = false;
                        break;
                    }
                    const uint32_t dst = ring + s * stage_bytes;
                    if (WFMT == FMT_FP16) {
                        mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)(A_BYTES + b_bytes));
                        tma_load_2d(dst, &g.tm_w, kb * BK, wt * BM, full0 + s * 8, policy);
                    } else {
                        mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)b_bytes);  // the weight half comes from the expanding warps
                    }
                    tma_load_2d(dst + A_BYTES, &g.tm_x, kb * BK, tt * g_bn, full0 + s * 8, policy);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: one lane; accumulators alternate between two tensor-memory halves ----
        if (lane == 0) {
            const uint32_t idesc = instr_desc_f16(g_bn);
            // This one thread issues every MMA of the block, in order: whenever the tiles are narrow its instruction count
            // per K block is the kernel's pace.  So everything that depends on the ring slot (the two barriers, the two
            // descriptors) is stepped by a constant and reset when the ring wraps, not recomputed.
            int tl = 0, s = 0;
            uint32_t ph = 0;
            bool ok = true;
            const uint32_t a_lo0 = smem_desc_lo(ring), b_lo0 = smem_desc_lo(ring + A_BYTES), lo_step = (uint32_t)stage_bytes >> 4;
            uint32_t full_s = full0, empty_s = empty0, a_lo = a_lo0, b_lo = b_lo0;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tl) {
                const int acc = tl & 1;
                if (tl >= 2 && !mbar_wait_bounded(acc_empty0 + acc * 8, (uint32_t)(((tl >> 1) - 1) & 1))) {
                    *reinterpret_cast<volatile int*>(g_status) = 6;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * g_cols);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait_bounded(full_s, ph)) {
                        *reinterpret_cast<volatile int*>(g_status) = 4;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_f16(tmem_d, desc_of(a_lo + 2 * k), desc_of(b_lo + 2 * k), idesc, (uint32_t)((kb | k) != 0));
                    umma_commit(empty_s);  // the stage is free once these MMAs have read it
                    if (++s == g_stages) {
                        s = 0;
                        ph ^= 1u;
                        full_s = full0; empty_s = empty0; a_lo = a_lo0; b_lo = b_lo0;
                    } else {
                        full_s += 8; empty_s += 8; a_lo += lo_step; b_lo += lo_step;
                    }
                }
                umma_commit(acc_full0 + acc * 8);  // this tile's accumulator is complete
            }
        }
    } else if (WFMT != FMT_FP16 && warp == 2 + EPI_WARPS + DQ_WARPS) {
        // ---- packed-weight producer: runs g_raw_stages ahead of the expanding warps ----
        if (lane == 0) {
            const uint64_t policy = l2_policy_evict_first();
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int wt = tile / g_ntok;
                for (int sp = 0; sp * RAW_SPAN < nkb; ++sp, ++it) {
                    const int r = it % g_raw_stages;
                    if (it >= g_raw_stages && !mbar_wait_bounded(raw_empty0 + r * 8, (uint32_t)(((it / g_raw_stages) - 1) & 1))) {
                        *reinterpret_cast<volatile int*>(g_status) = 11;
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(raw_full0 + r * 8, (uint32_t)RAW_BYTES);
                    tma_load_2d(raw_ring + r * RAW_BYTES, &g.tm_w, sp * 128, wt * BM, raw_full0 + r * 8, policy);
                }
            }
        }
    } else if (WFMT != FMT_FP16 && warp >= 2 + EPI_WARPS) {
        // ---- expanding warps: packed stage -> fp16 rows in the operand's swizzled layout ----
        // Operand layout (K-major, 128-byte swizzle): row r of the stage at (r / 8) * 1024 + (r % 8) * 128,
        // its 16-byte piece c at ((c ^ (r % 8)) * 16).
        // The warps work as NGRP groups of four: group g expands the K blocks with kb % NGRP == g, so
        // NGRP K blocks are in conversion at any time and a group's round trip through the barriers is
        // hidden behind the other groups'.
        constexpr int GRP_THREADS = 4 * 32;
        const int dq = tid - (2 + EPI_WARPS) * 32;   // 0 .. DQ_WARPS * 32 - 1
        const int grp = dq / GRP_THREADS, dt = dq % GRP_THREADS;
        const int K32 = g.K / 32;
        const uint16_t* const q4s = g.q4_scale;
        int it = 0, rit = -1;   // operand stages and packed spans passed so far
        bool ok = true;
        constexpr int Q4_PASSES = BM * 2 / GRP_THREADS, I8_PASSES = BM * 4 / GRP_THREADS;
        // Q4: a thread expands the same Q4_PASSES weight rows and the same half (blk) of every K block
        // it handles, so its block scales are entries of those rows' scale vectors: one aligned
        // 16-byte load per row brings the eight scales of four K blocks, fetched four blocks ahead
        // (rows whose scale vector is not a multiple of 16 bytes take two-byte loads).
        const int q_blk = dt & 1;
        const bool q4_vec = (K32 % 8) == 0 && (reinterpret_cast<uintptr_t>(q4s) & 15) == 0;
        uint4 sv_cur[Q4_PASSES], sv_next[Q4_PASSES];
#pragma unroll
        for (int ps = 0; ps < Q4_PASSES; ++ps) sv_cur[ps] = sv_next[ps] = make_uint4(0, 0, 0, 0);
        auto load_group = [&](int tile, int grp8, int ps) {   // scales 8 grp8 .. 8 grp8 + 7 of row ((ps * GRP_THREADS + dt) >> 1)
            const int row = (tile / g_ntok) * BM + ((ps * GRP_THREADS + dt) >> 1);
            if (tile < ntiles && row < gN && grp8 * 8 < K32) return *reinterpret_cast<const uint4*>(q4s + (size_t)row * K32 + grp8 * 8);
            return make_uint4(0, 0, 0, 0);
        };
        if (WFMT == FMT_Q4 && q4_vec) {
#pragma unroll
            for (int ps = 0; ps < Q4_PASSES; ++ps) sv_next[ps] = load_group(blockIdx.x, 0, ps);
        }
        // A group expands the K block of every packed span whose place in the span is the group's number
        // (spans hold as many K blocks as there are groups), so a warp steps through spans, not K blocks:
        // the bookkeeping of the blocks it does not expand would otherwise cost more than the expansion.
        static_assert(WFMT == FMT_FP16 || RAW_SPAN == NGRP, "one K block of every span per group");
        // a thread expands the same rows and the same place of every span: its offsets inside a packed span and
        // inside an operand slot never change
        constexpr int NPASS = WFMT == FMT_INT8 ? I8_PASSES : Q4_PASSES;
        uint32_t src_off[NPASS], dst_off[NPASS][4];
#pragma unroll
        for (int ps = 0; ps < NPASS; ++ps) {
            const int task = ps * GRP_THREADS + dt;
            if (WFMT == FMT_INT8) {
                const int row = task >> 2, ch = task & 3;   // 16 codes = 16 k
                const uint32_t rbase = (uint32_t)((row >> 3) * 1024 + (row & 7) * 128), x7 = (uint32_t)(row & 7);
                src_off[ps] = rbase + (((uint32_t)(grp * 4 + ch) ^ x7) << 4);
                dst_off[ps][0] = rbase + (((uint32_t)(2 * ch) ^ x7) << 4);
                dst_off[ps][1] = rbase + (((uint32_t)(2 * ch + 1) ^ x7) << 4);
                dst_off[ps][2] = dst_off[ps][3] = 0;
            } else {
                const int row = task >> 1, blk = task & 1;  // 32 nibbles = one scale block
                const uint32_t rbase = (uint32_t)((row >> 3) * 1024 + (row & 7) * 128), x7 = (uint32_t)(row & 7);
                src_off[ps] = rbase + (((uint32_t)(grp * 2 + blk) ^ x7) << 4);
#pragma unroll
                for (int j = 0; j < 4; ++j) dst_off[ps][j] = rbase + (((uint32_t)(4 * blk + j) ^ x7) << 4);
            }
        }
        const int spans = (nkb + RAW_SPAN - 1) / RAW_SPAN;
        // ring positions and pass parities are stepped, not divided out: four divisions per K block and warp were a
        // visible share of the loop
        int tl = 0, it_prev = 0, s = 0, r = -1;
        uint32_t ph = 0, rph = 1;   // (it / g_stages) & 1 and (rit / g_raw_stages) & 1
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tl) {
            for (int sp = 0; sp < spans; ++sp) {
                ++rit;
                if (++r == g_raw_stages) r = 0;
                if (r == 0) rph ^= 1u;
                const int kb = sp * RAW_SPAN + grp;
                if (WFMT == FMT_Q4 && q4_vec) {
#pragma unroll
                    for (int ps = 0; ps < Q4_PASSES; ++ps) {
                        sv_cur[ps] = sv_next[ps];
                        sv_next[ps] = (sp + 1 < spans) ? load_group(tile, sp + 1, ps) : load_group(tile + (int)gridDim.x, 0, ps);
                    }
                }
                if (kb >= nkb) {   // a short last span: nothing of it for this group
                    __syncwarp();
                    if (lane == 0) mbar_arrive(raw_empty0 + r * 8);
                    continue;
                }
                it = tl * nkb + kb;
                s += it - it_prev;
                it_prev = it;
                while (s >= g_stages) {
                    s -= g_stages;
                    ph ^= 1u;
                }
                uint16_t sc[Q4_PASSES];
#pragma unroll
                for (int ps = 0; ps < Q4_PASSES; ++ps) sc[ps] = 0;
                if (WFMT == FMT_Q4) {
#pragma unroll
                    for (int ps = 0; ps < Q4_PASSES; ++ps) {
                        if (q4_vec) {
                            const int e = (kb & 3) * 2 + q_blk;   // entry of the current group of eight
                            const uint32_t w32 = e < 2 ? sv_cur[ps].x : e < 4 ? sv_cur[ps].y : e < 6 ? sv_cur[ps].z : sv_cur[ps].w;
                            sc[ps] = (uint16_t)((e & 1) ? (w32 >> 16) : (w32 & 0xFFFFu));
                        } else {
                            const int row = (tile / g_ntok) * BM + ((ps * GRP_THREADS + dt) >> 1), blk = kb * 2 + q_blk;
                            if (row < gN && blk < K32) sc[ps] = q4s[(size_t)row * K32 + blk];
                        }
                    }
                }
                // the packed span has landed (this group's first K block of the span), and the MMAs that
                // read this operand slot last are done
                if (!mbar_wait_bounded(raw_full0 + r * 8, rph) || (it >= g_stages && !mbar_wait_bounded(empty0 + s * 8, ph ^ 1u))) {
                    if (lane == 0) *reinterpret_cast<volatile int*>(g_status) = 10;
                    ok = false;
                    break;
                }
                const uint32_t a_addr = ring + s * stage_bytes, raw = raw_ring + r * RAW_BYTES;
                // all of the thread's packed pieces are read before the first conversion: the loads are
                // volatile (ordered among themselves and with the stores), so a load placed after a store
                // would wait for it and every pass would pay the shared-memory latency again
                if (WFMT == FMT_INT8) {
                    uint32_t w[I8_PASSES][4];
#pragma unroll
                    for (int ps = 0; ps < I8_PASSES; ++ps)
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[ps][0]), "=r"(w[ps][1]), "=r"(w[ps][2]), "=r"(w[ps][3]) : "r"(raw + src_off[ps]));
#pragma unroll
                    for (int ps = 0; ps < I8_PASSES; ++ps) {
                        uint32_t h[8];
                        int8x4_to_half2x2(w[ps][0], h[0], h[1]);
                        int8x4_to_half2x2(w[ps][1], h[2], h[3]);
                        int8x4_to_half2x2(w[ps][2], h[4], h[5]);
                        int8x4_to_half2x2(w[ps][3], h[6], h[7]);
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a_addr + dst_off[ps][0]), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a_addr + dst_off[ps][1]), "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]) : "memory");
                    }
                } else {
                    uint32_t w[Q4_PASSES][4];
#pragma unroll
                    for (int ps = 0; ps < Q4_PASSES; ++ps)
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[ps][0]), "=r"(w[ps][1]), "=r"(w[ps][2]), "=r"(w[ps][3]) : "r"(raw + src_off[ps]));
#pragma unroll
                    for (int ps = 0; ps < Q4_PASSES; ++ps) {
                        const __half sh = __ushort_as_half(sc[ps]);
                        const __half2 s2 = __halves2half2(sh, sh);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t p04, p15, p26, p37;
                            q4x8_to_half2x4(w[ps][j], p04, p15, p26, p37);   // (n0,n4) (n1,n5) (n2,n6) (n3,n7), exact codes
                            uint32_t o[4];
                            asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o[0]) : "r"(p04), "r"(p15));  // (n0, n1)
                            asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o[1]) : "r"(p26), "r"(p37));  // (n2, n3)
                            asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o[2]) : "r"(p04), "r"(p15));  // (n4, n5)
                            asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o[3]) : "r"(p26), "r"(p37));  // (n6, n7)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&o[e]), s2);  // fp16(code * scale)
                                o[e] = *reinterpret_cast<const uint32_t*>(&v);
                            }
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a_addr + dst_off[ps][j]), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
                        }
                    }
                }
                fence_async_smem();   // the MMA reads the operand through the async proxy
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full0 + s * 8);
                    mbar_arrive(raw_empty0 + r * 8);   // this warp is done with the span
                }
            }
        }
    } else {
        // ---- epilogue warps: warp w owns accumulator lanes 32 (w % 4) .. +31 ----
        const int q = warp & 3;
        int tl = 0, n_stores = 0;
        bool failed = false;
        const int g_out_box = min(g_bn, OUT_ROWS);
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tl) {
            const int wt = tile / g_ntok, tt = tile - wt * g_ntok;
            const int n0 = wt * BM, m0 = tt * g_bn, acc = tl & 1;
            if (!failed && !mbar_wait_bounded_warp(acc_full0 + acc * 8, (uint32_t)((tl >> 1) & 1))) {
                failed = true;
                if (lane == 0) *reinterpret_cast<volatile int*>(g_status) = 5;
            }
            tc_fence_after();
            if (!failed && g_tma_store) {
                // fast path: scale and convert, lay the tile out as [token][weight row] in shared
                // memory (a warp writes 64 contiguous bytes per token) and let one tensor store
                // write it; the tensor map clips the rows and columns past M and N.  For the
                // in-place residual the tile's current values are fetched into the same buffer
                // first; for a row-sharded gather the finished tile is also copied to the peers.
                const int n = n0 + q * 32 + lane;
                const float rs = (g_rs && n < gN) ? __half2float(__ushort_as_half(g_rs[n])) : 1.0f;
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * g_cols) + ((uint32_t)(q * 32) << 16);
                const uint32_t dst0 = out_stage + (uint32_t)((q * 32 + lane) * 2);
                // the tile leaves in slabs of at most OUT_ROWS tokens (the staging buffer's height)
                for (int h0 = 0; h0 < g_bn; h0 += OUT_ROWS) {
                    const int hrows = min(OUT_ROWS, g_bn - h0);
                    if (n_stores > 0) {
                        // the previous slab's store must have finished reading the staging buffer
                        if (warp == 2 && lane == 0) bulk_wait_read0();
                        asm volatile("bar.sync 2, %0;" ::"n"(EPI_WARPS * 32) : "memory");
                    }
                    if (g_epi == EPI_RESIDUAL) {
                        if (warp == 2 && lane == 0) {
                            mbar_arrive_expect_tx(res_bar, (uint32_t)(g_out_box * BM * 2));
                            tma_load_2d(out_stage, &g.tm_out, n0, m0 + h0, res_bar, l2_policy_evict_normal());
                        }
                        if (!mbar_wait_bounded_warp(res_bar, (uint32_t)(n_stores & 1))) {
                            failed = true;
                            if (lane == 0) *reinterpret_cast<volatile int*>(g_status) = 9;
                        }
                    }
                    for (int c = 0; c < hrows; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(tmem_d + (uint32_t)(h0 + c), r);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            float v = __uint_as_float(r[j]) * rs;
                            const uint32_t addr = dst0 + (uint32_t)((c + j) * (BM * 2));
                            if (g_epi == EPI_RESIDUAL) {
                                uint16_t old;
                                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(old) : "r"(addr) : "memory");
                                v = __half2float(__ushort_as_half(old)) + v;
                            }
                            const uint16_t hv = __half_as_ushort(__float2half_rn(v));
                            asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(hv) : "memory");
                        }
                    }
                    if (h0 + OUT_ROWS >= g_bn) {
                        // the accumulator is free as soon as its last columns have been read
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty0 + acc * 8);
                    }
                    fence_async_smem();
                    asm volatile("bar.sync 2, %0;" ::"n"(EPI_WARPS * 32) : "memory");
                    if (warp == 2 && lane == 0) tma_store_2d(&g.tm_out, out_stage, n0, m0 + h0);
                    ++n_stores;
                    if (g_npeer > 0) {
                        // peers get the slab in 16-byte pieces, 256 contiguous bytes per token row
                        const int et = (warp - 2) * 32 + lane;
                        const int rows = min(hrows, gM - m0 - h0);
                        for (int i = et; i < rows * 16; i += EPI_WARPS * 32) {
                            const int mr = i >> 4, ch = i & 15;
                            if (n0 + ch * 8 >= gN) continue;
                            uint4 v;
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                                         : "r"(out_stage + (uint32_t)(mr * (BM * 2) + ch * 16)) : "memory");
                            const size_t o = (size_t)(m0 + h0 + mr) * g_ld + n0 + ch * 8;
#pragma unroll
                            for (int p = 0; p < 7; ++p)
                                if (p < g_npeer) *reinterpret_cast<uint4*>(g_peer[p] + o) = v;
                        }
                    }
                }
                continue;
            }
            if (!failed) {
                const int n = n0 + q * 32 + lane;
                const float rs = (g_rs && n < gN) ? __half2float(__ushort_as_half(g_rs[n])) : 1.0f;
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * g_cols) + ((uint32_t)(q * 32) << 16);
                for (int c = 0; c < g_bn; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_d + (uint32_t)c, r);
                    if (n < gN) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int m = m0 + c + j;
                            if (m < gM && c + j < g_bn) {
                                float v = __uint_as_float(r[j]) * rs;
                                uint16_t* o = g_out + (size_t)m * g_ld + n;
                                if (g_epi == EPI_RESIDUAL) v = __half2float(__ushort_as_half(*o)) + v;
                                const uint16_t hv = __half_as_ushort(__float2half_rn(v));
                                *o = hv;
                                #pragma unroll
                                for (int p = 0; p < 7; ++p)
                                    if (p < g_npeer) g_peer[p][(size_t)m * g_ld + n] = hv;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + acc * 8);
        }
    }
    if (g_tma_store && warp == 2 && lane == 0) bulk_wait0();  // all of this block's tensor stores have landed
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)(2 * g_cols));
    if (tid == 0 && g.sig.world > 0) gather_signal_block_done(g.sig);
}

}  // namespace

cudaError_t gemm_tc_configure() {
    cudaError_t e = cudaFuncSetAttribute(linear_gemm_tc_kernel<FMT_FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(linear_gemm_tc_kernel<FMT_INT8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(linear_gemm_tc_kernel<FMT_Q4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

bool gemm_tc_supported(int fmt, int M, int N, int K, const void* x, const void* W, const void* out) {
    if (M <= 16 || N < 1 || K < 64 || (K % 8) != 0) return false;
    if (fmt == FMT_INT8 && K < 128) return false;   // every expanding group needs a K block in every tile
    if (fmt == FMT_Q4 && K < 256) return false;
    if (fmt == FMT_INT8 && (K % 16) != 0) return false;   // packed rows keep a 16-byte pitch for the tensor copies
    if (fmt == FMT_Q4 && (K % 32) != 0) return false;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return al16(x) && al16(W) && out != nullptr;
}

cudaError_t launch_gemm_tc(int fmt, const void* W, const uint16_t* scale, const uint16_t* x, uint16_t* out, int M, int N, int K,
                           int ld_out, int epi, int* status, uint16_t* const* peer_out, int npeer, const GatherSignal* sig, cudaStream_t st) {
    GemmK g;
    const uint16_t* row_scale = fmt == FMT_INT8 ? scale : nullptr;
    g.q4_scale = fmt == FMT_Q4 ? scale : nullptr;
    g.sig = GatherSignal{};
    if (sig) g.sig = *sig;
    if (npeer < 0 || npeer > 7) return cudaErrorInvalidValue;
    g.npeer = npeer;
    for (int p = 0; p < 7; ++p) g.peer_out[p] = p < npeer ? peer_out[p] : nullptr;
    // The epilogue goes through a staging tile in shared memory and one tensor store per tile
    // when the output rows keep 16-byte pitch and alignment (lane-by-lane stores otherwise).
    bool aligned = (ld_out % 8) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    for (int p = 0; p < npeer; ++p) aligned = aligned && (reinterpret_cast<uintptr_t>(peer_out[p]) & 15) == 0;
    g.tma_store = aligned ? 1 : 0;
    const int raw_bytes = fmt == FMT_FP16 ? 0 : BM * 128;  // packed spans: 128 bytes of each of the tile's rows
    // The groups of expanding warps fill consecutive operand slots at the same time, each waiting for "the MMAs that
    // read my slot one ring pass ago".  That wait is by phase parity, and it is only meaningful when the pass before
    // that one is certainly over, which the group knows from its own previous K block as long as the ring has at
    // least as many slots as there are groups (MMAs complete in order).  A ring shorter than the group count could let
    // a group pass a stale phase and overwrite a slot in use, so the token tile is narrowed until the ring is deep enough.
    const int min_stages = dq_warps(fmt) >= 4 ? dq_warps(fmt) / 4 : 2;
    const int bn_max = 256;
    int bn = M >= bn_max ? bn_max : ((M + 15) / 16) * 16;
    int b_bytes = 0, stage_bytes = 0, out_bytes = 0, raw_stages = 0, stages = 0;
    for (;;) {
        b_bytes = ((bn * BK * 2 + 1023) / 1024) * 1024;
        stage_bytes = A_BYTES + b_bytes;
        const int out_rows = bn < OUT_ROWS ? ((bn + 31) / 32) * 32 : OUT_ROWS;  // the epilogue reads 32 columns at a time
        out_bytes = g.tma_store ? out_rows * BM * 2 : 0;
        // packed weights get a ring of their own, deep enough to cover the HBM latency
        raw_stages = 0;
        if (raw_bytes) {
            raw_stages = 4;
            while (raw_stages > 2 && (227 * 1024 - 2048 - out_bytes - raw_stages * raw_bytes) / stage_bytes < (min_stages > 3 ? min_stages : 3)) --raw_stages;
        }
        stages = (227 * 1024 - 2048 - out_bytes - raw_stages * raw_bytes) / stage_bytes;
        if (stages > 6) stages = 6;
        if (stages >= (min_stages > 2 ? min_stages : 2) || bn <= 32) break;
        bn = (bn / 2 + 15) / 16 * 16;
    }
    if (stages < (min_stages > 2 ? min_stages : 2)) return cudaErrorInvalidValue;
    g.bn = bn;
    g.ntok = (M + bn - 1) / bn;
    g.tmem_cols = 32;
    while (g.tmem_cols < bn) g.tmem_cols *= 2;
    g.raw_stages = raw_stages;
    g.stages = stages;
    g.out = out;
    g.row_scale = row_scale;
    g.M = M; g.N = N; g.K = K; g.ld_out = ld_out;
    g.epi = epi;
    g.status = status;
    bool okw;
    if (fmt == FMT_FP16) okw = encode_tiled_2d(&g.tm_w, /*fp16*/ true, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, BK, BM);
    else if (fmt == FMT_INT8) okw = encode_tiled_2d(&g.tm_w, false, W, (uint64_t)K, (uint64_t)N, (uint64_t)K, 128, BM);
    else okw = encode_tiled_2d(&g.tm_w, false, W, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, 128, BM);
    if (!okw) return cudaErrorInvalidValue;
    if (!encode_tiled_2d(&g.tm_x, true, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, bn)) return cudaErrorInvalidValue;
    if (g.tma_store && !encode_tiled_2d(&g.tm_out, true, out, (uint64_t)N, (uint64_t)M, (uint64_t)ld_out * 2, BM, bn < OUT_ROWS ? bn : OUT_ROWS, /*swizzle128=*/false))
        return cudaErrorInvalidValue;
    const size_t smem = 2048 + (size_t)stages * stage_bytes + (size_t)raw_stages * raw_bytes + out_bytes;
    unsigned grid = (unsigned)(((N + BM - 1) / BM) * g.ntok);
    const unsigned sms = (unsigned)current_sm_count();
    if (grid > sms) grid = sms;  // persistent: one block per SM walks the tiles
    if (fmt == FMT_FP16) linear_gemm_tc_kernel<FMT_FP16><<<grid, GEMM_THREADS, smem, st>>>(g);
    else if (fmt == FMT_INT8) linear_gemm_tc_kernel<FMT_INT8><<<grid, gemm_threads(FMT_INT8), smem, st>>>(g);
    else linear_gemm_tc_kernel<FMT_Q4><<<grid, gemm_threads(FMT_Q4), smem, st>>>(g);
    return cudaGetLastError();
}

}  // namespace nnb
