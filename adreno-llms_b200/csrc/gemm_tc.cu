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
// int8 / Q4 weights take this path through an fp16 copy made by dequant_half_kernel
// (int8 codes are exact in fp16 and the per-row scale is applied in the epilogue, after
// the full-K sum, like the GEMV; Q4 stores code x block-scale rounded to fp16).
#include <cuda.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nnb {
namespace {

constexpr int BM = 128;       // weight rows per tile (UMMA M)
constexpr int BK = 64;        // K elements per stage = one 128-byte swizzle span of fp16
constexpr int EPI_WARPS = 4;
constexpr int GEMM_THREADS = (2 + EPI_WARPS) * 32;  // producer warp, MMA warp, four epilogue warps
constexpr int A_BYTES = BM * BK * 2;  // 16 KB

struct GemmK {
    alignas(64) CUtensorMap tm_w;  // [N][K] fp16, box 64 x 128
    alignas(64) CUtensorMap tm_x;  // [M][K] fp16, box 64 x BN
    alignas(64) CUtensorMap tm_out;  // [M][ld_out] fp16, box 128 x BN (dense), when tma_store
    int tma_store;                   // plain-store epilogue through shared memory and one tensor store per tile
    uint16_t* out;                 // [M][ld_out]
    const uint16_t* row_scale;     // int8 weights: fp16 scale per weight row, else null
    int M, N, K, ld_out;
    int bn;        // tokens per tile (multiple of 16, <= 256)
    int ntok;      // token tiles
    int stages;
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

__global__ void __launch_bounds__(GEMM_THREADS) linear_gemm_tc_kernel(const __grid_constant__ GemmK g) {
    extern __shared__ __align__(128) uint8_t smem[];
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
    const uint32_t res_bar = s_base + 176;
    const uint32_t ring = (s_base + 1024u + 1023u) & ~1023u;
    const int b_bytes = g_bn * BK * 2;
    const int stage_bytes = A_BYTES + ((b_bytes + 1023) / 1024) * 1024;
    const int nkb = (g.K + BK - 1) / BK;
    const uint32_t out_stage = ring + (uint32_t)(g_stages * stage_bytes);  // [BN][128] fp16 staging of one output tile
    const int ntiles = ((gN + BM - 1) / BM) * g_ntok;

    if (tid == 0) {
        for (int s = 0; s < g_stages; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, 1);
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
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int wt = tile / g_ntok, tt = tile - wt * g_ntok;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % g_stages;
                    if (it >= g_stages && !mbar_wait_bounded(empty0 + s * 8, (uint32_t)(((it / g_stages) - 1) & 1))) {
                        *reinterpret_cast<volatile int*>(g_status) = 3;
                        ok = false;
                        break;
                    }
                    const uint32_t dst = ring + s * stage_bytes;
                    mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)(A_BYTES + b_bytes));
                    tma_load_2d(dst, &g.tm_w, kb * BK, wt * BM, full0 + s * 8, policy);
                    tma_load_2d(dst + A_BYTES, &g.tm_x, kb * BK, tt * g_bn, full0 + s * 8, policy);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: one lane; accumulators alternate between two tensor-memory halves ----
        if (lane == 0) {
            const uint32_t idesc = instr_desc_f16(g_bn);
            int it = 0, tl = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tl) {
                const int acc = tl & 1;
                if (tl >= 2 && !mbar_wait_bounded(acc_empty0 + acc * 8, (uint32_t)(((tl >> 1) - 1) & 1))) {
                    *reinterpret_cast<volatile int*>(g_status) = 6;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * g_cols);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % g_stages;
                    if (!mbar_wait_bounded(full0 + s * 8, (uint32_t)((it / g_stages) & 1))) {
                        *reinterpret_cast<volatile int*>(g_status) = 4;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = ring + s * stage_bytes, b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_f16(tmem_d, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc, (uint32_t)((kb | k) != 0));
                    umma_commit(empty0 + s * 8);  // the stage is free once these MMAs have read it
                }
                umma_commit(acc_full0 + acc * 8);  // this tile's accumulator is complete
            }
        }
    } else {
        // ---- epilogue warps: warp w owns accumulator lanes 32 (w % 4) .. +31 ----
        const int q = warp & 3;
        int tl = 0;
        bool failed = false;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tl) {
            const int wt = tile / g_ntok, tt = tile - wt * g_ntok;
            const int n0 = wt * BM, m0 = tt * g_bn, acc = tl & 1;
            if (!failed && !mbar_wait_bounded(acc_full0 + acc * 8, (uint32_t)((tl >> 1) & 1))) {
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
                if (tl > 0) {
                    // the previous tile's store must have finished reading the staging buffer
                    if (warp == 2 && lane == 0) bulk_wait_read0();
                    asm volatile("bar.sync 2, %0;" ::"n"(EPI_WARPS * 32) : "memory");
                }
                if (g_epi == EPI_RESIDUAL) {
                    if (warp == 2 && lane == 0) {
                        mbar_arrive_expect_tx(res_bar, (uint32_t)(g_bn * BM * 2));
                        tma_load_2d(out_stage, &g.tm_out, n0, m0, res_bar, l2_policy_evict_normal());
                    }
                    if (!mbar_wait_bounded(res_bar, (uint32_t)(tl & 1))) {
                        failed = true;
                        if (lane == 0) *reinterpret_cast<volatile int*>(g_status) = 9;
                    }
                }
                const uint32_t dst0 = out_stage + (uint32_t)((q * 32 + lane) * 2);
                for (int c = 0; c < g_bn; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_d + (uint32_t)c, r);
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
                // the accumulator is free as soon as it has been read
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + acc * 8);
                fence_async_smem();
                asm volatile("bar.sync 2, %0;" ::"n"(EPI_WARPS * 32) : "memory");
                if (warp == 2 && lane == 0) tma_store_2d(&g.tm_out, out_stage, n0, m0);
                if (g_npeer > 0) {
                    // peers get the tile in 16-byte pieces, 256 contiguous bytes per token row
                    const int et = (warp - 2) * 32 + lane;
                    const int rows = min(g_bn, gM - m0);
                    for (int i = et; i < rows * 16; i += EPI_WARPS * 32) {
                        const int mr = i >> 4, ch = i & 15;
                        if (n0 + ch * 8 >= gN) continue;
                        uint4 v;
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                                     : "r"(out_stage + (uint32_t)(mr * (BM * 2) + ch * 16)) : "memory");
                        const size_t o = (size_t)(m0 + mr) * g_ld + n0 + ch * 8;
#pragma unroll
                        for (int p = 0; p < 7; ++p)
                            if (p < g_npeer) *reinterpret_cast<uint4*>(g_peer[p] + o) = v;
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

// fp16 copy of a quantised weight for the tensor-core path.
template <int FMT>
__global__ void dequant_half_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ scale, uint16_t* __restrict__ out, int N, int K) {
    const size_t total = (size_t)N * K / 8;  // 8 outputs per thread step
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t e = i * 8, n = e / K;
        const int k = (int)(e - n * K);
        uint16_t h[8];
        if (FMT == FMT_INT8) {
            const uint2 v = *reinterpret_cast<const uint2*>(W + e);
            const int8_t* q = reinterpret_cast<const int8_t*>(&v);
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = __half_as_ushort(__int2half_rn((int)q[j]));  // exact; scale goes to the epilogue
        } else {
            const uint32_t v = *reinterpret_cast<const uint32_t*>(W + n * (size_t)(K / 2) + (k >> 1));
            const float s = __half2float(__ushort_as_half(scale[n * (size_t)(K / 32) + (k >> 5)]));
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = __half_as_ushort(__float2half_rn((float)((int)((v >> (4 * j)) & 0xF) - 8) * s));
        }
        *reinterpret_cast<uint4*>(out + e) = *reinterpret_cast<const uint4*>(h);
    }
}

}  // namespace

cudaError_t gemm_tc_configure() {
    return cudaFuncSetAttribute(linear_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

bool gemm_tc_supported(int M, int N, int K, const void* x, const void* W, const void* out) {
    if (M <= 16 || N < 1 || K < 64 || (K % 8) != 0) return false;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return al16(x) && al16(W) && out != nullptr;
}

cudaError_t launch_dequant_half(int fmt, int N, int K, const void* W, const uint16_t* scale, uint16_t* out, cudaStream_t st) {
    const size_t total = (size_t)N * K / 8;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    if (fmt == FMT_INT8) dequant_half_kernel<FMT_INT8><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)W, scale, out, N, K);
    else dequant_half_kernel<FMT_Q4><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)W, scale, out, N, K);
    return cudaGetLastError();
}

cudaError_t launch_gemm_tc(const uint16_t* W_half, const uint16_t* row_scale, const uint16_t* x, uint16_t* out, int M, int N, int K,
                           int ld_out, int epi, int* status, uint16_t* const* peer_out, int npeer, const GatherSignal* sig, cudaStream_t st) {
    GemmK g;
    g.sig = GatherSignal{};
    if (sig) g.sig = *sig;
    if (npeer < 0 || npeer > 7) return cudaErrorInvalidValue;
    g.npeer = npeer;
    for (int p = 0; p < 7; ++p) g.peer_out[p] = p < npeer ? peer_out[p] : nullptr;
    int bn = M >= 256 ? 256 : ((M + 15) / 16) * 16;
    g.bn = bn;
    g.ntok = (M + bn - 1) / bn;
    g.tmem_cols = 32;
    while (g.tmem_cols < bn) g.tmem_cols *= 2;
    const int b_bytes = ((bn * BK * 2 + 1023) / 1024) * 1024;
    const int stage_bytes = A_BYTES + b_bytes;
    // The epilogue goes through a staging tile in shared memory and one tensor store per tile
    // when the output rows keep 16-byte pitch and alignment (lane-by-lane stores otherwise).
    bool aligned = (ld_out % 8) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    for (int p = 0; p < npeer; ++p) aligned = aligned && (reinterpret_cast<uintptr_t>(peer_out[p]) & 15) == 0;
    g.tma_store = aligned ? 1 : 0;
    const int out_bytes = g.tma_store ? ((bn + 31) / 32) * 32 * BM * 2 : 0;  // the epilogue reads 32 columns at a time
    int stages = (227 * 1024 - 2048 - out_bytes) / stage_bytes;
    if (stages > 6) stages = 6;
    if (stages < 2) return cudaErrorInvalidValue;
    g.stages = stages;
    g.out = out;
    g.row_scale = row_scale;
    g.M = M; g.N = N; g.K = K; g.ld_out = ld_out;
    g.epi = epi;
    g.status = status;
    if (!encode_tiled_2d(&g.tm_w, /*fp16*/ true, W_half, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, BK, BM)) return cudaErrorInvalidValue;
    if (!encode_tiled_2d(&g.tm_x, true, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, bn)) return cudaErrorInvalidValue;
    if (g.tma_store && !encode_tiled_2d(&g.tm_out, true, out, (uint64_t)N, (uint64_t)M, (uint64_t)ld_out * 2, BM, bn, /*swizzle128=*/false))
        return cudaErrorInvalidValue;
    const size_t smem = 2048 + (size_t)stages * stage_bytes + out_bytes;
    unsigned grid = (unsigned)(((N + BM - 1) / BM) * g.ntok);
    if (grid > 148u) grid = 148u;  // persistent: one block per SM walks the tiles
    linear_gemm_tc_kernel<<<grid, GEMM_THREADS, smem, st>>>(g);
    return cudaGetLastError();
}

}  // namespace nnb
