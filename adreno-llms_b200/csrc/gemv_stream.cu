// Weight-streaming linear kernel for decode (M <= 16), sm_100a.
//
// Replaces the reference's M == 1 OpenCL GEMV family behind pytorch_linear
//   fp16  src/models/lfm2-5-350m/kernels/gemv_m1.cl, src/models/qwen2-5-0-5b/kernels/gemv_m1.cl,
//         src/models/smollm2-135m-instruct/kernels/block_fused.cl
//   int8  src/models/lfm2-5-350m/kernels/gemv_m1_int8.cl,
//         src/models/smollm2-135m-instruct/kernels/block_fused_int8.cl
//   Q4    src/models/lfm2-5-350m/kernels/gemv_m1_q4.cl
// and their fused epilogues (residual add, SwiGLU of two weights, silu(gate) * W3 x,
// several weights sharing x).  The arithmetic contract is theirs: activations and
// outputs fp16, all sums in fp32, int8 scale applied once after the full-K sum,
// Q4 scale applied per 32-weight block, nibble value = nibble - 8.
//
// Design (HBM-bound work; the tensor cores are only there to take the FMAs off
// the issue slots so that the dequantisation fits beside a 6+ TB/s stream):
//   * a tile is 32 consecutive weight rows; a pipeline stage is `kcb` bytes of
//     each of those rows.  Every lane of a warp issues ONE bulk async copy
//     (cp.async.bulk, TMA unit) for its row into a padded shared-memory row, all
//     32 completing on the stage's mbarrier.  Each warp runs its own ring of
//     stages, so the SM keeps warps x (stages-1) x 32 x kcb bytes in flight and no
//     warp ever waits for another in the main loop.
//   * Q4 block scales travel with the stage through per-lane cp.async tracked by
//     the same mbarrier.
//   * weights go shared memory -> registers with ldmatrix, are converted to exact
//     fp16 integers in registers (prmt / lop3 magic numbers, no int->float
//     converts), and are multiplied with mma.sync m16n8k16 (fp32 accumulate)
//     against the activations, which sit in shared memory pre-permuted so that one
//     ldmatrix yields the B fragment matching the packed weight order.
//     M = 1..8 uses one n8 tile, M = 9..16 two; rows >= M read a zero block.
//   * small N: `kw` warps split K of one tile and reduce through shared memory in
//     a fixed order (deterministic).
//   * launched with programmatic dependent launch: the weight prefetch of launch
//     i+1 (weights never depend on activations) overlaps the tail of launch i;
//     only the activation staging waits for the prior grid.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdio>
#include <cstdlib>

#include "kernels.h"
#include "ptx.cuh"

namespace nnb {

namespace {

constexpr int TILE_ROWS = 32;
constexpr int MAX_WARPS = 8;
constexpr int HDR_BYTES = 128;  // 64 B of zeros + room for the mbarriers' alignment

__host__ __device__ inline int fmt_row_bytes(int fmt, int K) { return fmt == FMT_FP16 ? K * 2 : fmt == FMT_INT8 ? K : K / 2; }

struct Geo {  // shared-memory geometry, computed identically on host and device
    int nbox;         // 128-byte column boxes per stage (each 32 rows x 128 B = 4 KB, swizzled)
    int sstride;      // bytes between Q4 scale rows in a stage
    int stage_bytes;  // one stage of one warp (multiple of 1024)
    int xstride;      // bytes between activation rows
    int off_bar, off_x, off_red, off_ring;
    int total;
};

constexpr int BOX_BYTES = TILE_ROWS * 128;

__host__ __device__ inline Geo make_geo(int fmt, int M, int K, int kcb, int nwarps, int stages, int nt) {
    Geo g;
    g.nbox = (kcb + 127) / 128;
    g.sstride = kcb / 8 + 16;
    g.stage_bytes = g.nbox * BOX_BYTES + (fmt == FMT_Q4 ? ((TILE_ROWS * g.sstride + 1023) / 1024) * 1024 : 0);
    g.xstride = K * 2 + 16;
    g.off_bar = 64;
    g.off_x = HDR_BYTES + ((nwarps * stages * 8 + 127) / 128) * 128;
    g.off_red = g.off_x + ((M * g.xstride + 127) / 128) * 128;
    g.off_ring = ((g.off_red + nwarps * 32 * 2 * nt * 4 * 4 + 1023) / 1024) * 1024;
    g.total = g.off_ring + nwarps * stages * g.stage_bytes + 1024;  // slack to align the ring to 1 KB
    return g;
}

struct KArgs {
    alignas(64) CUtensorMap tm[4];  // weight views: seg[0..2], and W2 for the two-weight epilogue
    LinArgs a;
    int stages;
    int rowbytes;
    int nchunks;
    int evict_first;  // weights larger than L2 are streamed with an evict-first policy
#ifdef NNB_TRACE
    unsigned long long* trace;  // debug build only: per-launch phase timestamps
    int trace_slot;
    int dbg_mode;               // debug build only: 1 = no arithmetic, 2 = loads only, 3 = no MMA
#endif
};

#ifdef NNB_TRACE
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TRACE(i) do { } while (0)
#else
#define TRACE(i) do { } while (0)
#endif

// Stage the activations [M, K] fp16 into shared memory, permuted per format so
// that ldmatrix over 16-byte pieces yields B fragments in the weights' packed order:
//   fp16: identity
//   int8: per 16 k   -> [k 0,1,4,5,8,9,12,13][k 2,3,6,7,10,11,14,15]
//   Q4  : per 32 k   -> piece j, pair t = (k 8t+j, k 8t+j+4)
template <int FMT>
__device__ __forceinline__ void stage_x(const uint16_t* __restrict__ x, int M, int K, uint8_t* xs, int xstride, int tid,
                                        int nthreads) {
    if (FMT == FMT_FP16) {
        const int per_row = K / 8;  // 16-byte pieces
        for (int i = tid; i < M * per_row; i += nthreads) {
            const int m = i / per_row, p = i - m * per_row;
            const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * K + p * 8);
            *reinterpret_cast<uint4*>(xs + m * xstride + p * 16) = v;
        }
    } else if (FMT == FMT_INT8) {
        const int per_row = K / 16;
        for (int i = tid; i < M * per_row; i += nthreads) {
            const int m = i / per_row, p = i - m * per_row;
            const uint4 a = *reinterpret_cast<const uint4*>(x + (size_t)m * K + p * 16);
            const uint4 b = *reinterpret_cast<const uint4*>(x + (size_t)m * K + p * 16 + 8);
            uint4 lo, hi;  // words are k pairs: a = (0,1)(2,3)(4,5)(6,7), b = (8,9)...(14,15)
            lo.x = a.x; lo.y = a.z; lo.z = b.x; lo.w = b.z;
            hi.x = a.y; hi.y = a.w; hi.z = b.y; hi.w = b.w;
            *reinterpret_cast<uint4*>(xs + m * xstride + p * 32) = lo;
            *reinterpret_cast<uint4*>(xs + m * xstride + p * 32 + 16) = hi;
        }
    } else {
        const int per_row = K / 32;
        for (int i = tid; i < M * per_row; i += nthreads) {
            const int m = i / per_row, p = i - m * per_row;
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)m * K + p * 32);
            uint32_t o[4][4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint4 v = src[t];  // k 8t .. 8t+7 as pairs (0,1)(2,3)(4,5)(6,7)
                o[0][t] = __byte_perm(v.x, v.z, 0x5410);  // (k0, k4)
                o[1][t] = __byte_perm(v.x, v.z, 0x7632);  // (k1, k5)
                o[2][t] = __byte_perm(v.y, v.w, 0x5410);  // (k2, k6)
                o[3][t] = __byte_perm(v.y, v.w, 0x7632);  // (k3, k7)
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(xs + m * xstride + p * 64 + j * 16) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
        }
    }
}

template <int FMT, int NT, bool DUAL>
__global__ void __launch_bounds__(MAX_WARPS * 32) linear_stream_kernel(const __grid_constant__ KArgs ka) {
    extern __shared__ __align__(128) uint8_t smem[];
    const LinArgs& a = ka.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nwarps = blockDim.x >> 5;
    const int stages = ka.stages;
    const int kcb = a.kcb, kw = a.kw;
    const int rowbytes = ka.rowbytes, nchunks = ka.nchunks;
    const Geo geo = make_geo(FMT, a.M, a.K, kcb, nwarps, stages, NT);

    const uint32_t s_base = smem_u32(smem);
    const uint32_t zero_addr = s_base;
    const uint32_t bar0 = s_base + geo.off_bar + warp * stages * 8;
    uint8_t* xs = smem + geo.off_x;
    float* red = reinterpret_cast<float*>(smem + geo.off_red);
    const uint32_t ring = ((s_base + geo.off_ring + 1023u) & ~1023u) + warp * stages * geo.stage_bytes;

    TRACE(0);
    if (tid < 16) reinterpret_cast<uint32_t*>(smem)[tid] = 0u;
    if (lane == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(bar0 + s * 8, FMT == FMT_Q4 ? 33u : 1u);
        mbar_init_fence();
    }
    __syncwarp();

    // ---- this warp's work: tiles (slot-strided) x its share of the K chunks ----
    const int slots = nwarps / kw;
    const int tslot = warp / kw, kpart = warp - tslot * kw;
    const int my_chunks = (nchunks - kpart + kw - 1) / kw;
    const int tile_first = blockIdx.x * slots + tslot;
    const int tile_step = gridDim.x * slots;
    const int my_tiles = tile_first < a.ntiles ? (a.ntiles - tile_first + tile_step - 1) / tile_step : 0;
    const int n_items = my_tiles * my_chunks;

    const uint64_t policy = ka.evict_first ? l2_policy_evict_first() : l2_policy_evict_normal();
    auto issue = [&](int it) {
        const int ti = it / my_chunks, cj = it - ti * my_chunks;
        const int tile = tile_first + ti * tile_step;
        const int c = kpart + cj * kw;
        const int stage = it % stages;
        const uint32_t bar = bar0 + stage * 8;
        const uint32_t dst = ring + stage * geo.stage_bytes;
        const int cb = min(kcb, rowbytes - c * kcb);
        // One elected lane drives the TMA unit: per 128-byte column of the chunk, one tiled
        // tensor copy of 32 rows (two of 16 rows for the two-weight epilogue) into a
        // 128-byte-swizzled 4 KB box.  Rows past the end of the weight arrive as zeros.
        const int nb = (cb + 127) >> 7;
        int sg = 0, row0;
        if (DUAL) {
            row0 = tile * 16;
        } else {
            if (a.nseg > 1 && tile >= a.seg[1].tile0) sg = 1;
            if (a.nseg > 2 && tile >= a.seg[2].tile0) sg = 2;
            row0 = (tile - a.seg[sg].tile0) * TILE_ROWS;
        }
        if (lane == 0) {
            mbar_arrive_expect_tx(bar, (uint32_t)(nb * BOX_BYTES));
            for (int b = 0; b < nb; ++b) {
                if (DUAL) {
                    tma_load_2d(dst + b * BOX_BYTES, &ka.tm[0], c * kcb + b * 128, row0, bar, policy);
                    tma_load_2d(dst + b * BOX_BYTES + BOX_BYTES / 2, &ka.tm[3], c * kcb + b * 128, row0, bar, policy);
                } else {
                    tma_load_2d(dst + b * BOX_BYTES, &ka.tm[sg], c * kcb + b * 128, row0, bar, policy);
                }
            }
        }
        if (FMT == FMT_Q4) {
            // block scales of this lane's row ride along through cp.async on the same mbarrier
            const uint16_t* sbase;
            int row;
            if (DUAL) {
                row = min(row0 + (lane & 15), a.seg[0].N - 1);
                sbase = lane < 16 ? a.seg[0].scale : a.scale2;
            } else {
                row = min(row0 + lane, a.seg[sg].N - 1);
                sbase = a.seg[sg].scale;
            }
            const uint8_t* ssrc = reinterpret_cast<const uint8_t*>(sbase) + ((size_t)row * (a.K / 32)) * 2 + (size_t)c * (kcb / 8);
            const uint32_t sdst = dst + geo.nbox * BOX_BYTES + lane * geo.sstride;
            const int sb = cb / 8;
            if (((reinterpret_cast<uintptr_t>(ssrc) | (uintptr_t)sb) & 15) == 0) {
                for (int o = 0; o < sb; o += 16) cp_async_16(sdst + o, ssrc + o);
            } else {
                for (int o = 0; o < sb; o += 4) cp_async_4(sdst + o, ssrc + o);
            }
            cp_async_mbar_arrive_noinc(bar);
        }
    };

    // Weight prefetch does not depend on the previous launch: start it first.
    const int pre = min(stages - 1, n_items);
    for (int it = 0; it < pre; ++it) issue(it);

    // ---- per-lane fragment addressing ----
    const int g = lane >> 2, t = lane & 3;
    // A operands live in swizzled boxes: 16-byte piece q of row r sits at
    //   box(q / 8) + r * 128 + ((q % 8) ^ (r % 8)) * 16.
    // fp16 / int8 ldmatrix.x4: matrices = (rows 0-7, piece q) (rows 8-15, q) (rows 0-7, q+1) (rows 8-15, q+1)
    const uint32_t a_row_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * 128);
    const uint32_t a_q_lane = (uint32_t)(lane >> 4);
    // Q4 ldmatrix.x4: matrices = the four 8-row groups of one 16-byte piece
    const uint32_t aq_row_off = (uint32_t)(lane * 128);
    const uint32_t xr = (uint32_t)(lane & 7);
    auto piece_addr = [&](uint32_t sw, uint32_t row_off, uint32_t q) {
        return sw + (q >> 3) * BOX_BYTES + row_off + (((q & 7) ^ xr) << 4);
    };
    // B: matrix j = lane/8 (16-byte piece j of the 32-k step), row n = lane%8 (+8 per n tile)
    uint32_t b_base[NT], b_step[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int n = (lane & 7) + nt * 8;
        const bool valid = n < a.M;
        b_base[nt] = valid ? smem_u32(xs) + n * geo.xstride + (lane >> 3) * 16 : zero_addr;
        b_step[nt] = valid ? 64u : 0u;
    }

    // Two accumulator sets per row block: consecutive k steps alternate between them so
    // that the tensor-core results of one step are not on the critical path of the next.
    float acc[2][2][NT][4];
    float sc_reg[2][2];          // int8: row scales of the current tile (rows g, g+8 of each block)
    float res_reg[2][2][NT][2];  // in-place epilogues: the values to be updated
    bool failed = false;

    auto tile_segment = [&](int tile) {
        int si = 0;
        if (a.nseg > 1 && tile >= a.seg[1].tile0) si = 1;
        if (a.nseg > 2 && tile >= a.seg[2].tile0) si = 2;
        return si;
    };
    // Per-row scales do not depend on the previous launch: fetch them ahead of use.
    auto prefetch_scales = [&](int tile) {
        if (FMT != FMT_INT8) return;
        if (DUAL) {
#pragma unroll
            for (int i2 = 0; i2 < 2; ++i2) {
                const int n = min(tile * 16 + g + i2 * 8, a.seg[0].N - 1);
                sc_reg[0][i2] = __half2float(__ushort_as_half(a.seg[0].scale[n]));
                sc_reg[1][i2] = __half2float(__ushort_as_half(a.scale2[n]));
            }
        } else {
            const LinSeg& sg = a.seg[tile_segment(tile)];
            const int row0 = (tile - sg.tile0) * TILE_ROWS;
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int i2 = 0; i2 < 2; ++i2)
                    sc_reg[rb][i2] = __half2float(__ushort_as_half(sg.scale[min(row0 + rb * 16 + g + i2 * 8, sg.N - 1)]));
        }
    };
    if (my_tiles > 0 && kpart == 0) prefetch_scales(tile_first);

    TRACE(1);
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    TRACE(2);
    stage_x<FMT>(a.x, a.M, a.K, xs, geo.xstride, tid, blockDim.x);
    __syncthreads();
    TRACE(3);

    const uint32_t rb_stride = 16 * 128;

#ifdef NNB_TRACE
    long long cyc_issue = 0, cyc_wait = 0, cyc_comp = 0, cyc_epi = 0, cyc_t0 = clock64(), cyc_a, cyc_b;
#define CYC_BEGIN() cyc_a = clock64()
#define CYC_END(acc) do { cyc_b = clock64(); acc += cyc_b - cyc_a; cyc_a = cyc_b; } while (0)
#else
#define CYC_BEGIN() do { } while (0)
#define CYC_END(acc) do { } while (0)
#endif
    for (int it = 0; it < n_items; ++it) {
        const int ti = it / my_chunks, cj = it - ti * my_chunks;
        const int tile = tile_first + ti * tile_step;
        const int c = kpart + cj * kw;
        CYC_BEGIN();
        if (cj == 0) {
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[u][rb][nt][i] = 0.f;
            if (kpart == 0) {
                if (ti > 0) prefetch_scales(tile);
                if (!DUAL && (a.epi == EPI_RESIDUAL || a.epi == EPI_SILU_GATE)) {
                    const LinSeg& sg = a.seg[tile_segment(tile)];
                    const int row0 = (tile - sg.tile0) * TILE_ROWS;
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for (int i2 = 0; i2 < 2; ++i2)
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                                for (int j = 0; j < 2; ++j) {
                                    const int n = row0 + rb * 16 + g + i2 * 8, m = nt * 8 + 2 * t + j;
                                    res_reg[rb][i2][nt][j] = (n < sg.N && m < a.M)
                                        ? __half2float(__ushort_as_half(sg.out[(size_t)m * sg.ld_out + n])) : 0.f;
                                }
                }
            }
        }
        __syncwarp();  // every lane is done reading the stage that is about to be refilled
        if (it + stages - 1 < n_items) issue(it + stages - 1);
        CYC_END(cyc_issue);

        const int stage = it % stages;
        // A wait that runs out records an error and skips the arithmetic from then on;
        // the warp still walks its items so that the block's barriers stay matched.
        if (!failed && !mbar_wait_bounded(bar0 + stage * 8, (uint32_t)((it / stages) & 1))) {
            failed = true;
            if (lane == 0) *reinterpret_cast<volatile int*>(a.status) = 1;
        }
        const uint32_t sw = ring + stage * geo.stage_bytes;
#ifdef NNB_TRACE
        const int cb = (failed || ka.dbg_mode == 1) ? 0 : min(kcb, rowbytes - c * kcb);
#else
        const int cb = failed ? 0 : min(kcb, rowbytes - c * kcb);
#endif
        if (it == 0) TRACE(4);
        CYC_END(cyc_wait);

        if (FMT == FMT_FP16) {
            // one step = 64 bytes of each row = 32 k = two MMAs per row block
            auto step = [&](int s, float (&ac)[2][NT][4]) {
                uint32_t b[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) ldsm_x4(b_base[nt] + s * b_step[nt], b[nt][0], b[nt][1], b[nt][2], b[nt][3]);
                uint32_t av[2][2][4];
                const uint32_t q = (uint32_t)(s - (c * kcb) / 64) * 4 + a_q_lane;
                const uint32_t ap0 = piece_addr(sw, a_row_off, q), ap1 = piece_addr(sw, a_row_off, q + 2);
#pragma unroll
                for (int rb = 0; rb < 2; ++rb) {
                    ldsm_x4(ap0 + rb * rb_stride, av[rb][0][0], av[rb][0][1], av[rb][0][2], av[rb][0][3]);
                    ldsm_x4(ap1 + rb * rb_stride, av[rb][1][0], av[rb][1][1], av[rb][1][2], av[rb][1][3]);
                }
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                            mma_16816(ac[rb][nt], av[rb][h][0], av[rb][h][1], av[rb][h][2], av[rb][h][3], b[nt][2 * h], b[nt][2 * h + 1]);
            };
            const int s0 = (c * kcb) / 64, s1 = s0 + cb / 64;
            int s = s0;
            for (; s + 2 <= s1; s += 2) {
                step(s, acc[0]);
                step(s + 1, acc[1]);
            }
            if (s < s1) step(s, acc[0]);
        } else if (FMT == FMT_INT8) {
            // one step = 32 bytes of each row = 32 k = two MMAs per row block
            auto step = [&](int s, float (&ac)[2][NT][4]) {
                uint32_t b[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) ldsm_x4(b_base[nt] + s * b_step[nt], b[nt][0], b[nt][1], b[nt][2], b[nt][3]);
                uint32_t w[2][4];
                const uint32_t ap = piece_addr(sw, a_row_off, (uint32_t)(s - (c * kcb) / 32) * 2 + a_q_lane);
#pragma unroll
                for (int rb = 0; rb < 2; ++rb) ldsm_x4(ap + rb * rb_stride, w[rb][0], w[rb][1], w[rb][2], w[rb][3]);
#ifdef NNB_TRACE
                if (ka.dbg_mode == 2) {
                    ac[0][0][0] += __uint_as_float((w[0][0] ^ w[1][1] ^ b[0][0]) & 0x3f800000u);
                    return;
                }
#endif
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb) {
                        uint32_t h01, h23, k01, k23;
                        int8x4_to_half2x2(w[rb][2 * h], h01, h23);
                        int8x4_to_half2x2(w[rb][2 * h + 1], k01, k23);
#ifdef NNB_TRACE
                        if (ka.dbg_mode == 3) {
                            ac[rb][0][0] += __uint_as_float((h01 ^ k01 ^ h23 ^ k23 ^ b[0][2 * h]) & 0x3f800000u);
                            continue;
                        }
#endif
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_16816(ac[rb][nt], h01, k01, h23, k23, b[nt][2 * h], b[nt][2 * h + 1]);
                    }
            };
            const int s0 = (c * kcb) / 32, s1 = s0 + cb / 32;
            int s = s0;
            for (; s + 4 <= s1; s += 4) {
                step(s, acc[0]);
                step(s + 1, acc[1]);
                step(s + 2, acc[0]);
                step(s + 3, acc[1]);
            }
            for (; s < s1; ++s) {
                if (s & 1) step(s, acc[1]);
                else step(s, acc[0]);
            }
        } else {
            // one step = 16 bytes of each row = one 32-weight block = two MMAs per row block,
            // summed from zero and folded in with the block's scale
            const uint8_t* sc = smem + (sw - s_base) + geo.nbox * BOX_BYTES;
            const int g0 = (c * kcb) / 16;
            auto step = [&](int s, float (&ac)[2][NT][4]) {
                uint32_t b[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) ldsm_x4(b_base[nt] + s * b_step[nt], b[nt][0], b[nt][1], b[nt][2], b[nt][3]);
                uint32_t w[4];
                ldsm_x4(piece_addr(sw, aq_row_off, (uint32_t)(s - g0)), w[0], w[1], w[2], w[3]);
#pragma unroll
                for (int rb = 0; rb < 2; ++rb) {
                    uint32_t p04, p15, p26, p37, q04, q15, q26, q37;
                    q4x8_to_half2x4(w[rb * 2], p04, p15, p26, p37);
                    q4x8_to_half2x4(w[rb * 2 + 1], q04, q15, q26, q37);
                    const float s_lo = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(sc + (rb * 16 + g) * geo.sstride + (s - g0) * 2)));
                    const float s_hi = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(sc + (rb * 16 + g + 8) * geo.sstride + (s - g0) * 2)));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        float d[4] = {0.f, 0.f, 0.f, 0.f};
                        mma_16816(d, p04, q04, p15, q15, b[nt][0], b[nt][1]);
                        mma_16816(d, p26, q26, p37, q37, b[nt][2], b[nt][3]);
                        ac[rb][nt][0] = fmaf(d[0], s_lo, ac[rb][nt][0]);
                        ac[rb][nt][1] = fmaf(d[1], s_lo, ac[rb][nt][1]);
                        ac[rb][nt][2] = fmaf(d[2], s_hi, ac[rb][nt][2]);
                        ac[rb][nt][3] = fmaf(d[3], s_hi, ac[rb][nt][3]);
                    }
                }
            };
            const int s1 = g0 + cb / 16;
            int s = g0;
            for (; s + 4 <= s1; s += 4) {
                step(s, acc[0]);
                step(s + 1, acc[1]);
                step(s + 2, acc[0]);
                step(s + 3, acc[1]);
            }
            for (; s < s1; ++s) {
                if (s & 1) step(s, acc[1]);
                else step(s, acc[0]);
            }
        }

        CYC_END(cyc_comp);
        if (cj != my_chunks - 1) continue;
        if (ti == 0) TRACE(5);

        // ---- tile finished: fold the two accumulator sets, combine the K parts (fixed
        //      order), then the epilogue ----
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[0][rb][nt][i] += acc[1][rb][nt][i];
        if (kw > 1) {
            float* mine = red + (warp * 32 + lane) * (2 * NT * 4);
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) mine[(rb * NT + nt) * 4 + i] = acc[0][rb][nt][i];
            asm volatile("bar.sync %0, %1;" ::"r"(1 + tslot), "r"(kw * 32) : "memory");
            if (kpart == 0) {
                for (int p = 1; p < kw; ++p) {
                    const float* o = red + ((warp + p) * 32 + lane) * (2 * NT * 4);
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[0][rb][nt][i] += o[(rb * NT + nt) * 4 + i];
                }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + tslot), "r"(kw * 32) : "memory");
        }
        if (kpart != 0) continue;

        if (DUAL) {
            const LinSeg& sg = a.seg[0];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = tile * 16 + g + (i >> 1) * 8;
                    const int m = nt * 8 + 2 * t + (i & 1);
                    if (n < sg.N && m < a.M) {
                        float gv = acc[0][0][nt][i], uv = acc[0][1][nt][i];
                        if (FMT == FMT_INT8) {
                            gv *= sc_reg[0][i >> 1];
                            uv *= sc_reg[1][i >> 1];
                        }
                        const float r = (gv / (1.0f + expf(-gv))) * uv;
                        sg.out[(size_t)m * sg.ld_out + n] = __half_as_ushort(__float2half_rn(r));
                    }
                }
        } else {
            const LinSeg& sg = a.seg[tile_segment(tile)];
            const int row0 = (tile - sg.tile0) * TILE_ROWS;
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int i2 = 0; i2 < 2; ++i2) {
                    const int n = row0 + rb * 16 + g + i2 * 8;
                    if (n >= sg.N) continue;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int m = nt * 8 + 2 * t + j;
                            if (m >= a.M) continue;
                            float v = acc[0][rb][nt][i2 * 2 + j];
                            if (FMT == FMT_INT8) v *= sc_reg[rb][i2];
                            if (a.epi == EPI_RESIDUAL) {
                                v = res_reg[rb][i2][nt][j] + v;
                            } else if (a.epi == EPI_SILU_GATE) {
                                const float gt = res_reg[rb][i2][nt][j];
                                v = gt * (1.0f / (1.0f + expf(-gt))) * v;
                            }
                            sg.out[(size_t)m * sg.ld_out + n] = __half_as_ushort(__float2half_rn(v));
                        }
                }
        }
    }
#ifdef NNB_TRACE
    cyc_epi = clock64() - cyc_t0 - cyc_issue - cyc_wait - cyc_comp;
    if (ka.trace && lane == 0 && blockIdx.x < 32) {
        unsigned long long* o = ka.trace + ((size_t)ka.trace_slot * 32 + blockIdx.x) * 8 * 8 + warp * 8;
        o[0] = cyc_issue; o[1] = cyc_wait; o[2] = cyc_comp; o[3] = cyc_epi; o[4] = n_items; o[5] = clock64() - cyc_t0;
    }
#endif
}

template <int FMT, int NT, bool DUAL>
cudaError_t launch_t(const KArgs& ka, const StreamPlan& p, int nwarps, cudaStream_t st, bool pdl) {
    auto kern = linear_stream_kernel<FMT, NT, DUAL>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.grid);
    cfg.blockDim = dim3((unsigned)(nwarps * 32));
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, ka);
}

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

#ifdef NNB_TRACE
unsigned long long* g_trace = nullptr;
int g_trace_slots = 0, g_trace_next = 0;
#endif

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;

// 2-D byte view of a weight: [rows][rowbytes], box = 128 bytes x box_rows rows, 128-byte swizzle.
bool make_weight_map(CUtensorMap* m, const void* W, int rows, int rowbytes, int box_rows) {
    if (!g_encode_tiled) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)rowbytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)rowbytes};
    const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    return g_encode_tiled(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(W), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int FMT, int NT, bool DUAL>
cudaError_t configure_one() {
    return cudaFuncSetAttribute(linear_stream_kernel<FMT, NT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

}  // namespace

cudaError_t stream_configure() {
    cudaError_t e;
    if (!g_encode_tiled) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (!fn || q != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        g_encode_tiled = (EncodeTiledFn)fn;
    }
#define CFG(F, N, D) if ((e = configure_one<F, N, D>()) != cudaSuccess) return e;
    CFG(FMT_FP16, 1, false) CFG(FMT_FP16, 2, false) CFG(FMT_FP16, 1, true) CFG(FMT_FP16, 2, true)
    CFG(FMT_INT8, 1, false) CFG(FMT_INT8, 2, false) CFG(FMT_INT8, 1, true) CFG(FMT_INT8, 2, true)
    CFG(FMT_Q4, 1, false) CFG(FMT_Q4, 2, false) CFG(FMT_Q4, 1, true) CFG(FMT_Q4, 2, true)
#undef CFG
    return cudaSuccess;
}

// Shapes the streaming kernel takes: 1 <= M <= 16, rows of at least 128 bytes whose
// length is a multiple of 64 bytes (fp16: K % 32, int8: K % 64, Q4: K % 128), and
// 16-byte aligned operands.  Everything else goes to the generic kernel.
bool stream_supported(int fmt, int M, int K, const LinArgs& a) {
    if (M < 1 || M > 16) return false;
    const int rb = fmt_row_bytes(fmt, K);
    if (rb < 128 || (rb % 64) != 0) return false;
    if (fmt == FMT_Q4 && (K % 64) != 0) return false;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    for (int i = 0; i < a.nseg; ++i) {
        if (!al16(a.seg[i].W)) return false;
        if (fmt == FMT_Q4 && (reinterpret_cast<uintptr_t>(a.seg[i].scale) & 3)) return false;
    }
    if (a.epi == EPI_SWIGLU && (!al16(a.W2) || (fmt == FMT_Q4 && (reinterpret_cast<uintptr_t>(a.scale2) & 3)))) return false;
    if (!al16(a.x)) return false;
    return true;
}

// Geometry heuristics (environment overrides NNB_KCB / NNB_KW / NNB_WARPS / NNB_STAGES /
// NNB_CTAS are for tuning runs):
//   * kcb: the row is cut into equal chunks of at most ~512 bytes (a multiple of 64);
//   * few tiles: the warps of a block split K (kw) so the whole operator is requested at once;
//   * warps and stages are sized so that about three blocks fit one SM.
StreamPlan stream_plan(int fmt, int M, int K, int ntiles, int sm_count, size_t smem_limit) {
    StreamPlan p = {};
    const int rb = fmt_row_bytes(fmt, K);
    const int nt = M > 8 ? 2 : 1;
    // stage width: whole 128-byte columns (the TMA box width), default 256 bytes per row
    int target = env_int("NNB_KCB", 256);
    target = target < 128 ? 128 : target > 1024 ? 1024 : (target / 128) * 128;
    int kcb = target;
    const int rb_cols = ((rb + 127) / 128) * 128;
    if (kcb > rb_cols) kcb = rb_cols;
    int stages = env_int("NNB_STAGES", 2);
    if (stages < 2 || stages > 8) stages = 2;
    int nwarps = env_int("NNB_WARPS", 0);
    if (nwarps != 1 && nwarps != 2 && nwarps != 4 && nwarps != 8) {
        // largest of {4, 2, 1} that lets three blocks share an SM
        nwarps = 4;
        while (nwarps > 1 && (size_t)make_geo(fmt, M, K, kcb, nwarps, stages, nt).total * 3 + 3072 > smem_limit) nwarps /= 2;
    }
    int kw = env_int("NNB_KW", 0);
    if (kw != 1 && kw != 2 && kw != 4 && kw != 8) {
        const int want = sm_count * 8;
        kw = 1;
        while (kw < nwarps && ntiles * kw < want) kw *= 2;
    }
    if (kw > nwarps) kw = nwarps;
    while (kw > 1 && (rb + kcb - 1) / kcb < kw) {
        // not enough chunks to share: cut the row finer if that is possible, else share less
        if (kcb > 128) kcb -= 128;
        else kw /= 2;
    }
    Geo g = make_geo(fmt, M, K, kcb, nwarps, stages, nt);
    while ((size_t)g.total > smem_limit && nwarps > 1) {
        nwarps /= 2;
        if (kw > nwarps) kw = nwarps;
        g = make_geo(fmt, M, K, kcb, nwarps, stages, nt);
    }
    while ((size_t)g.total > smem_limit && kcb > 128) {
        kcb -= 128;
        g = make_geo(fmt, M, K, kcb, nwarps, stages, nt);
    }
    if ((size_t)g.total > smem_limit) { p.ok = false; return p; }
    const int slots = nwarps / kw;
    int per_sm = (int)((smem_limit + 1024) / ((size_t)g.total + 1024));
    per_sm = per_sm < 1 ? 1 : per_sm > 6 ? 6 : per_sm;
    const int cap = env_int("NNB_CTAS", 0);
    if (cap > 0 && cap < per_sm) per_sm = cap;
    const int resident = sm_count * per_sm;
    const int need = (ntiles + slots - 1) / slots;
    p.grid = need < resident ? need : resident;
    if (p.grid < 1) p.grid = 1;
    p.kcb = kcb;
    p.kw = kw;
    p.warps = nwarps;
    p.stages = stages;
    p.smem = (size_t)g.total;
    p.ok = true;
    return p;
}

cudaError_t launch_stream(int fmt, const LinArgs& a, const StreamPlan& p, cudaStream_t st, bool pdl) {
    KArgs ka;
    ka.a = a;
    ka.a.kcb = p.kcb;
    ka.a.kw = p.kw;
    ka.stages = p.stages;
    ka.rowbytes = fmt_row_bytes(fmt, a.K);
    ka.nchunks = (ka.rowbytes + p.kcb - 1) / p.kcb;
    size_t wbytes = 0;
    for (int i = 0; i < a.nseg; ++i) wbytes += (size_t)a.seg[i].N * ka.rowbytes;
    ka.evict_first = wbytes > ((size_t)96 << 20) ? 1 : 0;
#ifdef NNB_TRACE
    ka.trace = g_trace;
    ka.trace_slot = g_trace_slots ? (g_trace_next++ % g_trace_slots) : 0;
    ka.dbg_mode = env_int("NNB_DBG_MODE", 0);
#endif
    const bool dual = a.epi == EPI_SWIGLU;
    const int nt = a.M > 8 ? 2 : 1;
    for (int i = 0; i < a.nseg; ++i)
        if (!make_weight_map(&ka.tm[i], a.seg[i].W, a.seg[i].N, ka.rowbytes, dual ? 16 : TILE_ROWS)) return cudaErrorInvalidValue;
    if (dual && !make_weight_map(&ka.tm[3], a.W2, a.seg[0].N, ka.rowbytes, 16)) return cudaErrorInvalidValue;
#define GO(F)                                                                              \
    if (fmt == F) {                                                                        \
        if (dual) return nt == 2 ? launch_t<F, 2, true>(ka, p, p.warps, st, pdl) : launch_t<F, 1, true>(ka, p, p.warps, st, pdl); \
        return nt == 2 ? launch_t<F, 2, false>(ka, p, p.warps, st, pdl) : launch_t<F, 1, false>(ka, p, p.warps, st, pdl);       \
    }
    GO(FMT_FP16) GO(FMT_INT8) GO(FMT_Q4)
#undef GO
    return cudaErrorInvalidValue;
}

#ifdef NNB_TRACE
extern "C" void nnb_debug_set_trace(void* buf, int slots) {
    g_trace = (unsigned long long*)buf;
    g_trace_slots = slots;
    g_trace_next = 0;
}
#endif

}  // namespace nnb
