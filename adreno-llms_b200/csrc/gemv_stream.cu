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
// Design (HBM-bound work; the tensor cores only take the FMAs off the issue slots so
// that the dequantisation fits beside a 6+ TB/s stream):
//   * a block = one producer warp + four consumer warps.  The producer's elected lane
//     drives the TMA unit: per pipeline stage it issues tiled tensor copies
//     (cp.async.bulk.tensor.2d, 128-byte swizzle) of 128 weight rows x 128-byte columns,
//     completing on the stage's "full" mbarrier; consumers hand a stage back through its
//     "empty" mbarrier.  Consumers never issue copies, so their issue slots go to
//     arithmetic only.
//   * each consumer warp owns 32 of the stage's rows (or, for operators with few rows,
//     the four warps split K of the same 32 rows and reduce through shared memory in a
//     fixed order).  Weights go shared memory -> registers with ldmatrix out of the
//     swizzled boxes (conflict-free, no padding), are converted to exact fp16 integers in
//     registers (prmt / lop3 magic numbers), and are multiplied with mma.sync m16n8k16
//     (fp32 accumulate) against the activations, which sit in shared memory pre-permuted
//     so that one ldmatrix yields the B fragment in the packed weight order.
//     M = 1..8 uses one n8 tile, M = 9..16 two; rows >= M read a zero block.
//   * Q4 block scales ride along on the same full barrier: one dense tensor copy per stage when
//     the scale rows keep a 16-byte pitch (K a multiple of 256), per-lane cp.async otherwise.
//   * launched with programmatic dependent launch: the producer never waits for the prior
//     grid (weights do not depend on activations), so the weight stream of launch i+1
//     starts under the tail of launch i; only the activation staging waits.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdio>
#include <cstdlib>

#include "kernels.h"
#include "plan.h"
#include "ptx.cuh"
#include "stream_core.cuh"

namespace nnb {

namespace {

constexpr int THREADS = STREAM_THREADS;

struct Geo {  // shared-memory geometry, computed identically on host and device
    int nbox;         // 128-byte column boxes per stage
    int sstride;      // bytes between Q4 scale rows in a stage
    int stage_bytes;  // one stage (multiple of 1024)
    int xstride;      // bytes between activation rows
    int off_bar, off_x, off_ctab, off_norm, off_red, off_ring;
    int total;
};

__host__ __device__ inline Geo make_geo(int fmt, int M, int K, int kcb, int stages, int nt, bool norm) {
    Geo g;
    g.nbox = stage_nbox(kcb);
    g.sstride = stage_sstride(kcb);
    g.stage_bytes = stage_bytes_of(fmt, kcb);
    g.xstride = x_stride_of(fmt, K);
    g.off_bar = 64;  // full[stages], empty[stages]
    g.off_x = HDR_BYTES + ((stages * 16 + 127) / 128) * 128;
    g.off_ctab = g.off_x + x_bytes_of(fmt, M, K);
    // fused RMSNorm: the normalised fp16 activations [M][K], from which the staging then reads
    g.off_norm = g.off_ctab + ctab_bytes_of(fmt, M, K);
    g.off_red = g.off_norm + (norm ? ((M * K * 2 + 127) / 128) * 128 : 0);
    g.off_ring = ((g.off_red + red_bytes_of(nt) + 1023) / 1024) * 1024;  // two reduction buffers
    g.total = g.off_ring + stages * g.stage_bytes + 1024;  // slack to align the ring to 1 KB
    return g;
}

struct KArgs {
    alignas(64) CUtensorMap tm[4];  // weight views: seg[0..2], and W2 for the two-weight epilogue
    LinArgs a;
    int stages;
    int rowbytes;
    int nchunks;      // K chunks of kcb bytes per row
    int evict_first;  // weights larger than L2 are streamed with an evict-first policy
    int scale_tma;    // Q4: block scales arrive by tensor copies (KArgsQ4::tm_s) instead of per-lane cp.async
};
// Only the Q4 kernels carry the scale views: kernel parameters are read by every block of every
// launch, and the small per-layer operators are launch-latency-bound.
struct KArgsQ4 : KArgs {
    alignas(64) CUtensorMap tm_s[4];  // Q4 scale views [N][K/16 bytes]: seg[0..2], and scale2
};
// The tensor maps travel in a kernel parameter of their own: their address is taken (the TMA unit
// reads them in place), and everything that shares a parameter with them would be read through
// generic loads; the scalars go by value in a second parameter and are read as constants.
struct KMaps { alignas(64) CUtensorMap tm[4]; };
struct KMapsQ4 { alignas(64) CUtensorMap tm[4]; alignas(64) CUtensorMap tm_s[4]; };
template <int FMT> struct KMapsFor { typedef KMaps type; };
template <> struct KMapsFor<FMT_Q4> { typedef KMapsQ4 type; };
struct KScal {
    LinArgs a;
    int stages, rowbytes, nchunks, evict_first, scale_tma;
};
__device__ __forceinline__ const CUtensorMap* scale_map(const KMaps&, int) { return nullptr; }
__device__ __forceinline__ const CUtensorMap* scale_map(const KMapsQ4& km, int i) { return &km.tm_s[i]; }
template <int FMT> struct KArgsFor { typedef KArgs type; };
template <> struct KArgsFor<FMT_Q4> { typedef KArgsQ4 type; };


// VAR selects how much of the kernel is compiled in: 0 = the plain projection, 1 = plus the RMSNorm
// prologue, 2 = plus the rarer features (balanced item dealing, peer stores, the gather signal,
// the fused arg-max).  The plain instantiation carries none of that code: the per-layer operators
// are launch-latency-bound, and every instruction-cache line their blocks have to fetch shows up
// in the step time (the full variant is 0.5 us slower per small launch with nothing switched on).
// ONE: the launch has a single activation row (decode).  The row count then is a compile-time
// constant and the multi-row staging loops and epilogues drop out of the instantiation, which the
// launch-latency-bound decode step feels as instruction-cache footprint.
template <int FMT, int NT, bool DUAL, int VAR, bool ONE>
__global__ void __launch_bounds__(THREADS) linear_stream_kernel(const __grid_constant__ typename KMapsFor<FMT>::type km, const KScal ka) {
    constexpr bool EXT = VAR == 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const LinArgs& a = ka.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Scalars used all over the kernel are read from the parameter block once.  The block's
    // address is taken (the tensor maps in it are handed to the TMA unit), so the compiler must
    // assume that any store may change it and would otherwise re-read a field after every store.
    const int aM = ONE ? 1 : a.M, aK = a.K, a_epi = a.epi, a_nseg = a.nseg;
    int* const a_status = a.status;
    const int seg1_tile0 = a.seg[1].tile0, seg2_tile0 = a.seg[2].tile0;
    const int stages = ka.stages, kcb = a.kcb;
    const bool ksplit = a.kw > 1;  // the four consumers split K of one 32-row tile
    const int rowbytes = ka.rowbytes, nchunks = ka.nchunks;
    const bool a_norm = VAR >= 1 && a.norm_w != nullptr;
    const Geo geo = make_geo(FMT, aM, aK, kcb, stages, NT, a_norm);
    const int warp_rows = DUAL ? 16 : WARP_ROWS;                       // rows of each weight per warp
    const int tile_rows = ksplit ? warp_rows : NCW * warp_rows;        // rows of each weight per block tile
    const int groups = ksplit ? (nchunks + NCW - 1) / NCW : nchunks;   // pipeline items per tile

    const uint32_t s_base = smem_u32(smem);
    const uint32_t zero_addr = s_base;
    const uint32_t full0 = s_base + geo.off_bar, empty0 = full0 + stages * 8;
    uint8_t* xs = smem + geo.off_x;
    float* red = reinterpret_cast<float*>(smem + geo.off_red);
    const uint32_t ring = (s_base + geo.off_ring + 1023u) & ~1023u;

    if (tid < 16) reinterpret_cast<uint32_t*>(smem)[tid] = 0u;
    if (FMT == FMT_INT8 && tid >= 32 && tid < 48) reinterpret_cast<uint32_t*>(xs + 3 * aM * geo.xstride)[tid - 32] = 0u;  // per-row max words
    const uint32_t xbar = s_base + geo.off_x - 8;  // batched calls: the staged activations have landed
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full0 + s * 8, (FMT == FMT_Q4 && !ka.scale_tma) ? 1u + NCW * 32u : 1u);
            mbar_init(empty0 + s * 8, (uint32_t)NCW);
        }
        if (!ONE) mbar_init(xbar, 1u);
        mbar_init_fence();
    }
    __syncthreads();

    // Pipeline items of this block.  Plain: whole tiles b, b + G, ... .  Balanced: a contiguous
    // share of the launch's tiles x groups items, which may begin and end inside a tile.
    const bool sk = EXT && a.streamk != 0;
    const long long sk_total = (long long)a.ntiles * groups;
    int n_items, tile_first, cg_first;
    if (sk) {
        const long long i0 = (long long)blockIdx.x * sk_total / (long long)gridDim.x;
        const long long i1 = (long long)(blockIdx.x + 1) * sk_total / (long long)gridDim.x;
        n_items = (int)(i1 - i0);
        tile_first = (int)(i0 / groups);
        cg_first = (int)(i0 - (long long)tile_first * groups);
    } else {
        const int my_tiles = (int)blockIdx.x < a.ntiles ? (a.ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
        n_items = my_tiles * groups;
        tile_first = (int)blockIdx.x;
        cg_first = 0;
    }
    const int tile_step = sk ? 1 : (int)gridDim.x;

    auto tile_segment = [&](int tile) {
        int si = 0;
        if (a_nseg > 1 && tile >= seg1_tile0) si = 1;
        if (a_nseg > 2 && tile >= seg2_tile0) si = 2;
        return si;
    };
    // A segment's fields by value.  The three cases index the parameter block with constants:
    // a run-time index would turn every field access into a generic-address load of a few
    // hundred cycles instead of a constant-bank read.
    auto seg_at = [&](int si) {
        LinSeg r;
        if (si == 0) r = a.seg[0];
        else if (si == 1) r = a.seg[1];
        else r = a.seg[2];
        return r;
    };

    // ================= producer warp: one elected lane feeds the TMA unit =================
    if (warp == NCW) {
        pdl_launch_dependents();
        if (lane == 0) {
            const uint64_t policy = ka.evict_first ? l2_policy_evict_first() : l2_policy_evict_normal();
            int tile_s = tile_first, cg = cg_first, stage = 0;
            for (int it = 0; it < n_items; ++it) {
                const int tile = tile_s;
                if (it >= stages && !mbar_wait_bounded(empty0 + stage * 8, (uint32_t)(((it / stages) - 1) & 1))) {
                    *reinterpret_cast<volatile int*>(a_status) = 2;
                    break;
                }
                const uint32_t dst = ring + stage * geo.stage_bytes, bar = full0 + stage * 8;
                const int sg = DUAL ? 0 : tile_segment(tile);
                const int row0 = (tile - (DUAL ? 0 : seg_at(sg).tile0)) * tile_rows;
                if (!ksplit) {
                    // one copy per 128-byte column covers the rows of all four consumers
                    const int cb = min(kcb, rowbytes - cg * kcb);
                    const int nb = (cb + 127) >> 7;
                    const bool stma = FMT == FMT_Q4 && ka.scale_tma;
                    const int bw = kcb / 8;  // bytes of block scales per row and stage
                    mbar_arrive_expect_tx(bar, (uint32_t)(nb * CTA_BOX + (stma ? NCW * WARP_ROWS * bw : 0)));
                    if (stma) {
                        const uint32_t sdst = dst + geo.nbox * CTA_BOX;
                        if (DUAL) {
                            tma_load_2d(sdst, scale_map(km, 0), cg * bw, row0, bar, policy);
                            tma_load_2d(sdst + (NCW * WARP_ROWS / 2) * bw, scale_map(km, 3), cg * bw, row0, bar, policy);
                        } else {
                            tma_load_2d(sdst, scale_map(km, sg), cg * bw, row0, bar, policy);
                        }
                    }
                    for (int b = 0; b < nb; ++b) {
                        const int x = cg * kcb + b * 128;
                        if (DUAL) {
                            tma_load_2d(dst + b * CTA_BOX, &km.tm[0], x, row0, bar, policy);
                            tma_load_2d(dst + b * CTA_BOX + CTA_BOX / 2, &km.tm[3], x, row0, bar, policy);
                        } else {
                            tma_load_2d(dst + b * CTA_BOX, &km.tm[sg], x, row0, bar, policy);
                        }
                    }
                } else {
                    // the consumers take consecutive K chunks of the same rows
                    const bool stma = FMT == FMT_Q4 && ka.scale_tma;
                    const int bw = kcb / 8;
                    uint32_t bytes = 0;
                    for (int w = 0; w < NCW; ++w) {
                        const int c = cg * NCW + w;
                        if (c < nchunks) bytes += (uint32_t)(((min(kcb, rowbytes - c * kcb) + 127) >> 7) * BOX_BYTES + (stma ? WARP_ROWS * bw : 0));
                    }
                    mbar_arrive_expect_tx(bar, bytes);
                    for (int w = 0; w < NCW; ++w) {
                        const int c = cg * NCW + w;
                        if (c >= nchunks) break;
                        if (stma) {
                            const uint32_t sdst = dst + geo.nbox * CTA_BOX;
                            if (DUAL) {
                                tma_load_2d(sdst + w * (WARP_ROWS / 2) * bw, scale_map(km, 0), c * bw, row0, bar, policy);
                                tma_load_2d(sdst + (NCW * WARP_ROWS / 2 + w * (WARP_ROWS / 2)) * bw, scale_map(km, 3), c * bw, row0, bar, policy);
                            } else {
                                tma_load_2d(sdst + w * WARP_ROWS * bw, scale_map(km, sg), c * bw, row0, bar, policy);
                            }
                        }
                        const int nb = (min(kcb, rowbytes - c * kcb) + 127) >> 7;
                        for (int b = 0; b < nb; ++b) {
                            const int x = c * kcb + b * 128;
                            if (DUAL) {
                                tma_load_2d(dst + b * CTA_BOX + w * (BOX_BYTES / 2), &km.tm[0], x, row0, bar, policy);
                                tma_load_2d(dst + b * CTA_BOX + CTA_BOX / 2 + w * (BOX_BYTES / 2), &km.tm[3], x, row0, bar, policy);
                            } else {
                                tma_load_2d(dst + b * CTA_BOX + w * BOX_BYTES, &km.tm[sg], x, row0, bar, policy);
                            }
                        }
                    }
                }
                if (++cg == groups) { cg = 0; tile_s += tile_step; }
                if (++stage == stages) stage = 0;
            }
        }
        return;
    }

    // ================= consumer warps =================
    const int g = lane >> 2, t = lane & 3;
    LaneGeo<NT> lg;
    lane_geo_init<FMT, NT>(lg, DUAL, warp, lane, aM, smem_u32(xs), geo.xstride, zero_addr, smem + geo.off_ctab);
    const float* rowscale = reinterpret_cast<const float*>(xs + 3 * aM * geo.xstride + 64);

    // rows of this warp inside its tile, and which warp writes results
    const int wrow_off = ksplit ? 0 : warp * warp_rows;
    const bool writer = !ksplit || warp == 0;

    float acc[2][2][NT][4];      // [accumulator set][row block][n tile][frag]
    int iacc[FMT == FMT_INT8 ? 3 : 1][2][NT][4];  // int8: exact integer sums per activation limb
    // Prefetched epilogue operands stay as raw fp16 bits until they are used, so that the
    // loads' latency is not waited for where they are issued.
    uint16_t sc_reg[2][2];          // int8: row scales of the current tile (rows g, g+8 of each block)
    // Single-token launches (one weight): lane L of a warp finishes row L of the warp's 32 rows, so
    // it prefetches one scale and one residual value and the tile leaves in one 64-byte store.
    const bool lane_rows = !DUAL && aM == 1;
    uint16_t sc1 = 0, res1 = 0;
    uint32_t res_reg[2][2][NT][2];  // in-place epilogues: the values to be updated
    bool failed = false;
    unsigned long long am_best = 0ull;  // fused arg-max: best key among this thread's rows

    // Per-row scales do not depend on the previous launch: fetch them ahead of use.
    auto prefetch_scales = [&](int tile) {
        if (FMT != FMT_INT8) return;
        if (DUAL) {
            if (aM == 1) {   // lane L (< 16) finishes row L of the warp's 16 rows
                const int n = min(tile * tile_rows + wrow_off + (lane & 15), a.seg[0].N - 1);
                sc1 = a.seg[0].scale[n];
                res1 = a.scale2[n];   // the up weight's scale rides in the spare register
                return;
            }
#pragma unroll
            for (int i2 = 0; i2 < 2; ++i2) {
                const int n = min(tile * tile_rows + wrow_off + g + i2 * 8, a.seg[0].N - 1);
                sc_reg[0][i2] = a.seg[0].scale[n];
                sc_reg[1][i2] = a.scale2[n];
            }
        } else {
            const LinSeg sg = seg_at(tile_segment(tile));
            const int row0 = (tile - sg.tile0) * tile_rows + wrow_off;
            if (lane_rows) {
                sc1 = sg.scale[min(row0 + lane, sg.N - 1)];
                return;
            }
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int i2 = 0; i2 < 2; ++i2)
                    sc_reg[rb][i2] = sg.scale[min(row0 + rb * 16 + g + i2 * 8, sg.N - 1)];
        }
    };
    // Q4: this lane's row of block scales for pipeline item `j` travels by cp.async and
    // arrives on the stage's full barrier (every lane arrives for every item).
    auto issue_scales = [&](int j) {
        const int lin = cg_first + j, ti = lin / groups, cg = lin - ti * groups;
        const int tile = tile_first + ti * tile_step;
        const int c = ksplit ? cg * NCW + warp : cg;
        const int stage = j % stages;
        const uint32_t bar = full0 + stage * 8;
        if (c < nchunks) {
            const uint16_t* sbase;
            int row;
            if (DUAL) {
                row = min(tile * tile_rows + wrow_off + (lane & 15), a.seg[0].N - 1);
                sbase = lane < 16 ? a.seg[0].scale : a.scale2;
            } else {
                const LinSeg sg = seg_at(tile_segment(tile));
                row = min((tile - sg.tile0) * tile_rows + wrow_off + lane, sg.N - 1);
                sbase = sg.scale;
            }
            const int cb = min(kcb, rowbytes - c * kcb);
            const uint8_t* ssrc = reinterpret_cast<const uint8_t*>(sbase) + ((size_t)row * (aK / 32)) * 2 + (size_t)c * (kcb / 8);
            const uint32_t sdst = ring + stage * geo.stage_bytes + geo.nbox * CTA_BOX + (warp * WARP_ROWS + lane) * geo.sstride;
            const int sb = cb / 8;
            if (((reinterpret_cast<uintptr_t>(ssrc) | (uintptr_t)sb) & 15) == 0) {
                for (int o = 0; o < sb; o += 16) cp_async_16(sdst + o, ssrc + o);
            } else {
                for (int o = 0; o < sb; o += 4) cp_async_4(sdst + o, ssrc + o);
            }
        }
        cp_async_mbar_arrive_noinc(bar);
    };

    // In-place epilogues read the values they update; issued early, used at the tile's end.
    auto prefetch_residual = [&](int tile) {
        if (DUAL || !(a_epi == EPI_RESIDUAL || a_epi == EPI_SILU_GATE)) return;
        const LinSeg sg = seg_at(tile_segment(tile));
        const int row0 = (tile - sg.tile0) * tile_rows + wrow_off;
        if (lane_rows) {
            res1 = (row0 + lane < sg.N) ? sg.out[row0 + lane] : (uint16_t)0;
            return;
        }
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
#pragma unroll
            for (int i2 = 0; i2 < 2; ++i2)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int n = row0 + rb * 16 + g + i2 * 8, m = nt * 8 + 2 * t + j;
                        res_reg[rb][i2][nt][j] = (n < sg.N && m < aM) ? (uint32_t)sg.out[(size_t)m * sg.ld_out + n] : 0u;
                    }
    };

    if (FMT == FMT_Q4 && !ka.scale_tma) {
        const int pre = min(stages - 1, n_items);
        for (int j = 0; j < pre; ++j) issue_scales(j);
    }
    if (n_items > 0 && writer) prefetch_scales(tile_first);

    pdl_launch_dependents();
    pdl_wait_prior_grid();
    if (n_items > 0 && writer) prefetch_residual(tile_first);
    const uint16_t* x_src = a.x;
    if (!ONE && a.staged != nullptr) {
        // the launch before this one (stage_image_kernel) wrote the staged form of all M rows in this
        // kernel's shared-memory layout: one bulk copy instead of M rows converted by every block
        if (tid == 0) {
            mbar_arrive_expect_tx(xbar, a.staged_bytes);
            bulk_g2s(smem_u32(xs), a.staged, a.staged_bytes, xbar, l2_policy_evict_normal());
        }
        if (!mbar_wait_bounded(xbar, 0u)) *reinterpret_cast<volatile int*>(a_status) = 5;
    } else {
    if (a_norm) {
        // RMSNorm prologue: the normalised fp16 rows go to shared memory and the staging below
        // reads them from there
        uint16_t* xn = reinterpret_cast<uint16_t*>(smem + geo.off_norm);
        rmsnorm_rows(a.x, a.norm_w, a.norm_eps, aM, aK, xn, red, tid, lane, warp);
        x_src = xn;
    }
    if (FMT == FMT_INT8) stage_x_int8(x_src, aM, aK, xs, geo.xstride, tid, NCW * 32);
    else stage_x<FMT>(x_src, aM, aK, xs, geo.xstride, reinterpret_cast<float*>(smem + geo.off_ctab), tid, NCW * 32);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");


    int tile_s = tile_first, cg = cg_first, ti = 0, stage = 0;
    uint32_t phase = 0;
    bool seg_has_head = true;  // the running sums began at the first K item of their tile
    for (int it = 0; it < n_items; ++it) {
        const int tile = tile_s;
        const int c = ksplit ? cg * NCW + warp : cg;
        const bool active = c < nchunks;
        if (cg == 0 || it == 0) {
            seg_has_head = (cg == 0);
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[u][rb][nt][i] = 0.f;
            if (FMT == FMT_INT8) {
#pragma unroll
                for (int l = 0; l < 3; ++l)
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int i = 0; i < 4; ++i) iacc[l % (FMT == FMT_INT8 ? 3 : 1)][rb][nt][i] = 0;
            }
            if (writer && it > 0) {
                prefetch_scales(tile);
                prefetch_residual(tile);
            }
        }
        if (FMT == FMT_Q4 && !ka.scale_tma) {
            __syncwarp();  // every lane is done with the scale rows that are about to be refilled
            if (it + stages - 1 < n_items) issue_scales(it + stages - 1);
        }
        // A wait that runs out records an error and skips the arithmetic from then on;
        // the warp still walks its items so that the block's barriers stay matched.
        if (!failed && !mbar_wait_bounded(full0 + stage * 8, phase)) {
            failed = true;
            if (lane == 0) *reinterpret_cast<volatile int*>(a_status) = 1;
        }
        const uint32_t sw = ring + stage * geo.stage_bytes;
        const int cb = (failed || !active) ? 0 : min(kcb, rowbytes - c * kcb);

        if constexpr (FMT == FMT_FP16) {
            chunk_fp16<NT>(lg, sw, c, kcb, cb, acc);
        } else if constexpr (FMT == FMT_INT8) {
            chunk_int8<NT>(lg, sw, c, kcb, cb, iacc);
        } else {
            // scale rows of this warp's two row blocks inside the stage's scale region: the
            // cp.async path keeps each warp's 32 rows together; tensor copies land whole boxes,
            // which for two weights means all gate rows first, then all up rows
            const int sstr = ka.scale_tma ? kcb / 8 : geo.sstride;
            const int srow0 = (ka.scale_tma && DUAL) ? warp * (WARP_ROWS / 2) : warp * WARP_ROWS;
            const int srow1 = (ka.scale_tma && DUAL) ? NCW * WARP_ROWS / 2 + warp * (WARP_ROWS / 2) : warp * WARP_ROWS + 16;
            const uint8_t* scb = smem + (sw - s_base) + geo.nbox * CTA_BOX;
            const uint8_t* const sc_rb[2] = {scb + (srow0 + g) * sstr, scb + (srow1 + g) * sstr};
            chunk_q4<NT>(lg, sw, c, kcb, cb, acc, sc_rb, sstr);
        }

        // hand the stage back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + stage * 8);
        if (++stage == stages) { stage = 0; phase ^= 1u; }
        const bool has_tail = (cg == groups - 1);              // this item ends its tile
        const bool seg_end = has_tail || it == n_items - 1;    // ... or this block's share of it
        if (++cg == groups) { cg = 0; tile_s += tile_step; }
        if (!seg_end) continue;
        ++ti;

        if constexpr (FMT == FMT_INT8) int8_recombine<NT>(iacc, acc[0], rowscale, aM, t);
        // ---- tile finished: fold the two accumulator sets, combine the K parts (fixed
        //      order), then the epilogue ----
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[0][rb][nt][i] += acc[1][rb][nt][i];
        if (ksplit) {
            // partial sums meet in shared memory; the buffer alternates between tiles so one
            // barrier per tile is enough
            float* buf = red + (ti & 1) * (NCW * 32 * 2 * NT * 4);
            if (warp != 0) {
                float* mine = buf + (warp * 32 + lane) * (2 * NT * 4);
#pragma unroll
                for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) mine[(rb * NT + nt) * 4 + i] = acc[0][rb][nt][i];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
            if (warp == 0) {
                for (int p = 1; p < NCW; ++p) {
                    const float* o = buf + (p * 32 + lane) * (2 * NT * 4);
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[0][rb][nt][i] += o[(rb * NT + nt) * 4 + i];
                }
            }
        }
        if (sk && !(seg_has_head && has_tail)) {
            float* part = a.sk_scratch + ((size_t)blockIdx.x * (NCW * 32) + (size_t)(warp * 32 + lane)) * (2 * NT * 4);
            if (!seg_has_head) {
                // the tile began in an earlier block: hand the sums over to it
                if (writer) {
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                            *reinterpret_cast<float4*>(part + (rb * NT + nt) * 4) =
                                make_float4(acc[0][rb][nt][0], acc[0][rb][nt][1], acc[0][rb][nt][2], acc[0][rb][nt][3]);
                }
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
                if (tid == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.sk_flags + blockIdx.x), "r"(1u) : "memory");
                continue;
            }
            // this block owns the tile but not its last K items: add the partial sums of the
            // blocks that follow, in block order (they produce theirs first thing)
            const long long tile_end = (long long)(tile + 1) * groups;
            for (int nb = (int)blockIdx.x + 1; nb < (int)gridDim.x; ++nb) {
                if ((long long)nb * sk_total / (long long)gridDim.x >= tile_end) break;
                if (tid == 0 && !failed) {
                    const long long t0 = clock64();
                    for (;;) {
                        unsigned v;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.sk_flags + nb) : "memory");
                        if (v) break;
                        if (clock64() - t0 > 400000000ll) {
                            *reinterpret_cast<volatile int*>(a_status) = 8;
                            break;
                        }
                        __nanosleep(40);
                    }
                    a.sk_flags[nb] = 0u;  // consumed; the flag is clear again for the next launch
                }
                asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
                if (writer) {
                    const float* o = a.sk_scratch + ((size_t)nb * (NCW * 32) + (size_t)(warp * 32 + lane)) * (2 * NT * 4);
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const float4 v = __ldcg(reinterpret_cast<const float4*>(o + (rb * NT + nt) * 4));
                            acc[0][rb][nt][0] += v.x;
                            acc[0][rb][nt][1] += v.y;
                            acc[0][rb][nt][2] += v.z;
                            acc[0][rb][nt][3] += v.w;
                        }
                }
            }
        }
        if (!writer) continue;

        if (DUAL) {
            const int seg_n = a.seg[0].N, seg_ld = a.seg[0].ld_out, m_count = aM;
            uint16_t* const seg_out = a.seg[0].out;
            if (m_count == 1) {
                // single token: rows g, g + 8 of the warp's 16 gate / up rows sit in lanes 0, 4, .. 28;
                // lane L < 16 takes row L and the 16 rows leave in one 32-byte store
                const int src = (lane & 7) * 4, hi = (lane >> 3) & 1;
                const float g0 = __shfl_sync(0xffffffffu, acc[0][0][0][0], src), g1 = __shfl_sync(0xffffffffu, acc[0][0][0][2], src);
                const float u0 = __shfl_sync(0xffffffffu, acc[0][1][0][0], src), u1 = __shfl_sync(0xffffffffu, acc[0][1][0][2], src);
                float gv = hi ? g1 : g0, uv = hi ? u1 : u0;
                const int n = tile * tile_rows + wrow_off + lane;
                if (lane < 16 && n < seg_n) {
                    if (FMT == FMT_INT8) {
                        gv *= __half2float(__ushort_as_half(sc1));
                        uv *= __half2float(__ushort_as_half(res1));
                    }
                    const float r = (gv / (1.0f + expf(-gv))) * uv;
                    seg_out[n] = __half_as_ushort(__float2half_rn(r));
                }
                continue;
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = tile * tile_rows + wrow_off + g + (i >> 1) * 8;
                    const int m = nt * 8 + 2 * t + (i & 1);
                    if (n < seg_n && m < m_count) {
                        float gv = acc[0][0][nt][i], uv = acc[0][1][nt][i];
                        if (FMT == FMT_INT8) {
                            gv *= __half2float(__ushort_as_half(sc_reg[0][i >> 1]));
                            uv *= __half2float(__ushort_as_half(sc_reg[1][i >> 1]));
                        }
                        const float r = (gv / (1.0f + expf(-gv))) * uv;
                        seg_out[(size_t)m * seg_ld + n] = __half_as_ushort(__float2half_rn(r));
                    }
                }
        } else {
            // Everything the store loop needs is copied into registers first: the segment lives in
            // kernel-parameter memory reached through a run-time index, and a 16-bit store may alias
            // it as far as the compiler can tell, so every field read after a store would be a fresh
            // (slow) load.
            const LinSeg sg = seg_at(tile_segment(tile));
            const int seg_n = sg.N, seg_ld = sg.ld_out, seg_tile0 = sg.tile0;
            uint16_t* const seg_out = sg.out;
            const int m_count = aM, epi = a_epi;
            const int npeer = EXT ? a.npeer : 0;
            unsigned long long* const am_slot = EXT ? a.argmax_slot : nullptr;
            const int am_base = EXT ? a.argmax_base : 0;
            uint16_t* peer[7];
#pragma unroll
            for (int p = 0; p < 7; ++p) peer[p] = (EXT && p < npeer) ? a.peer_out[p] : nullptr;
            const int row0 = (tile - seg_tile0) * tile_rows + wrow_off;
            if (lane_rows) {
                // the token's 32 results sit in lanes 0, 4, .. 28 (rows g, g + 8 of each row block):
                // bring row L to lane L, finish it there and store the 32 rows with one instruction
                const int src = (lane & 7) * 4, sel = lane >> 3;
                const float v00 = __shfl_sync(0xffffffffu, acc[0][0][0][0], src), v01 = __shfl_sync(0xffffffffu, acc[0][0][0][2], src);
                const float v10 = __shfl_sync(0xffffffffu, acc[0][1][0][0], src), v11 = __shfl_sync(0xffffffffu, acc[0][1][0][2], src);
                float v = sel == 0 ? v00 : sel == 1 ? v01 : sel == 2 ? v10 : v11;
                const int n = row0 + lane;
                if (n < seg_n) {
                    if (FMT == FMT_INT8) v = __fmul_rn(v, __half2float(__ushort_as_half(sc1)));  // roundings as in finish_row
                    if (EXT && sg.bias) v = __fadd_rn(__half2float(__float2half_rn(v)), __half2float(__ushort_as_half(sg.bias[n])));
                    if (epi == EPI_RESIDUAL) {
                        v = __fadd_rn(__half2float(__ushort_as_half(res1)), v);
                    } else if (epi == EPI_SILU_GATE) {
                        const float gt = __half2float(__ushort_as_half(res1));
                        v = gt * (1.0f / (1.0f + expf(-gt))) * v;
                    }
                    const uint16_t hv = __half_as_ushort(__float2half_rn(v));
                    if (!EXT || seg_out) seg_out[n] = hv;
                    if (EXT) {
#pragma unroll
                        for (int p = 0; p < 7; ++p)
                            if (p < npeer) peer[p][n] = hv;
                    }
                    if (EXT && am_slot && (hv & 0x7FFFu) <= 0x7C00u) {  // NaNs never win
                        const unsigned long long key = argmax_key_half(hv, am_base + n);
                        am_best = key > am_best ? key : am_best;
                    }
                }
                continue;
            }
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int i2 = 0; i2 < 2; ++i2) {
                    const int n = row0 + rb * 16 + g + i2 * 8;
                    if (n >= seg_n) continue;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int m = nt * 8 + 2 * t + j;
                            if (m >= m_count) continue;
                            float v = acc[0][rb][nt][i2 * 2 + j];
                            if (FMT == FMT_INT8) v = __fmul_rn(v, __half2float(__ushort_as_half(sc_reg[rb][i2])));  // roundings as in finish_row
                            if (EXT && sg.bias) v = __fadd_rn(__half2float(__float2half_rn(v)), __half2float(__ushort_as_half(sg.bias[n])));
                            if (epi == EPI_RESIDUAL) {
                                v = __fadd_rn(__half2float(__ushort_as_half((uint16_t)res_reg[rb][i2][nt][j])), v);
                            } else if (epi == EPI_SILU_GATE) {
                                const float gt = __half2float(__ushort_as_half((uint16_t)res_reg[rb][i2][nt][j]));
                                v = gt * (1.0f / (1.0f + expf(-gt))) * v;
                            }
                            const uint16_t hv = __half_as_ushort(__float2half_rn(v));
                            const size_t o = (size_t)m * seg_ld + n;
                            if (!EXT || seg_out) seg_out[o] = hv;
                            if (EXT) {
#pragma unroll
                                for (int p = 0; p < 7; ++p)
                                    if (p < npeer) peer[p][o] = hv;
                            }
                            if (EXT && am_slot && m == 0 && (hv & 0x7FFFu) <= 0x7C00u) {  // NaNs never win
                                const unsigned long long key = argmax_key_half(hv, am_base + n);
                                am_best = key > am_best ? key : am_best;
                            }
                        }
                }
        }
    }
    if (EXT && a.argmax_slot) {
        // fused arg-max: one atomic per warp, then the last block to finish publishes the index
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, am_best, o);
            am_best = other > am_best ? other : am_best;
        }
        if (lane == 0 && am_best) atomicMax(a.argmax_slot, am_best);
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        if (tid == 0) {
            const unsigned prev = atomicAdd(a.argmax_done, 1u);
            if (prev == gridDim.x - 1u) {
                __threadfence();
                const unsigned long long k = *reinterpret_cast<volatile unsigned long long*>(a.argmax_slot);
                *reinterpret_cast<volatile unsigned long long*>(a.argmax_slot) = 0ull;
                *reinterpret_cast<volatile unsigned*>(a.argmax_done) = 0u;
                if (a.sig.world > 0) {
                    // row-sharded pick: comm_pick_kernel chooses among the ranks' keys.  The words
                    // above are clear before the key can release the next launch that uses them.
                    __threadfence();
                    argmax_share_key(a.sig, k);
                } else {
                    *a.argmax_out = k ? (int)(0xFFFFFFFFu - (unsigned int)(k & 0xFFFFFFFFull)) : -1;
                }
            }
        }
    }
    if (EXT && a.sig.world > 0 && !a.argmax_slot) {
        // row-sharded gather: all of this block's outputs are stored; count the block in
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        if (tid == 0) gather_signal_block_done(a.sig);
    }
}

inline void fill_maps(KMaps& km, const KArgs& ka) {
    for (int i = 0; i < 4; ++i) km.tm[i] = ka.tm[i];
}
inline void fill_maps(KMapsQ4& km, const KArgsQ4& ka) {
    for (int i = 0; i < 4; ++i) { km.tm[i] = ka.tm[i]; km.tm_s[i] = ka.tm_s[i]; }
}

template <int FMT, int NT, bool DUAL, int VAR, bool ONE>
cudaError_t launch_o(const typename KArgsFor<FMT>::type& ka, const StreamPlan& p, cudaStream_t st, bool pdl) {
    auto kern = linear_stream_kernel<FMT, NT, DUAL, VAR, ONE>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.grid);
    cfg.blockDim = dim3((unsigned)THREADS);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    typename KMapsFor<FMT>::type km;
    fill_maps(km, ka);
    KScal ks;
    ks.a = ka.a;
    ks.stages = ka.stages; ks.rowbytes = ka.rowbytes; ks.nchunks = ka.nchunks; ks.evict_first = ka.evict_first; ks.scale_tma = ka.scale_tma;
    return cudaLaunchKernelEx(&cfg, kern, km, ks);
}

template <int FMT, int NT, bool DUAL, int VAR>
cudaError_t launch_e(const typename KArgsFor<FMT>::type& ka, const StreamPlan& p, cudaStream_t st, bool pdl) {
    if (NT == 1 && ka.a.M == 1) return launch_o<FMT, 1, DUAL, VAR, true>(ka, p, st, pdl);
    return launch_o<FMT, NT, DUAL, VAR, false>(ka, p, st, pdl);
}

template <int FMT, int NT, bool DUAL>
cudaError_t launch_t(const typename KArgsFor<FMT>::type& ka, const StreamPlan& p, cudaStream_t st, bool pdl) {
    const LinArgs& a = ka.a;
    const bool ext = a.streamk || a.npeer > 0 || a.sig.world > 0 || a.argmax_slot != nullptr || a.seg[0].out == nullptr ||
                     a.seg[0].bias != nullptr || a.seg[1].bias != nullptr || a.seg[2].bias != nullptr;
    if (ext) return launch_e<FMT, NT, DUAL, 2>(ka, p, st, pdl);
    if (a.norm_w) return launch_e<FMT, NT, DUAL, 1>(ka, p, st, pdl);
    return launch_e<FMT, NT, DUAL, 0>(ka, p, st, pdl);
}


typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;

// Encoding a tensor map costs the host about a microsecond, and a decode loop asks for the same
// few hundred (weight, tile) views token after token: keep them in a small direct-mapped,
// per-thread cache.  A map only describes (address, extents, box), so a hit is always valid.
struct MapSlot {
    const void* base;
    int rows, rowbytes, box_bytes, box_rows, swizzled;
    bool valid;
    CUtensorMap map;
};
constexpr int MAP_SLOTS = 2048;
thread_local MapSlot* t_map_cache = nullptr;

bool cached_byte_map(CUtensorMap* m, const void* base, int rows, int rowbytes, int box_bytes, int box_rows, bool swizzled) {
    if (!g_encode_tiled) return false;
    if (!t_map_cache) t_map_cache = new MapSlot[MAP_SLOTS]();
    uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
    h ^= (uint64_t)rows * 0x9E3779B97F4A7C15ull + (uint64_t)rowbytes * 0xC2B2AE3D27D4EB4Full + (uint64_t)(box_rows * 4 + box_bytes * 2 + (swizzled ? 1 : 0));
    MapSlot& s = t_map_cache[(h ^ (h >> 17) ^ (h >> 31)) % MAP_SLOTS];
    if (s.valid && s.base == base && s.rows == rows && s.rowbytes == rowbytes && s.box_bytes == box_bytes && s.box_rows == box_rows &&
        s.swizzled == (swizzled ? 1 : 0)) {
        *m = s.map;
        return true;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)rowbytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)rowbytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    if (g_encode_tiled(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                       swizzled ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    s.base = base; s.rows = rows; s.rowbytes = rowbytes; s.box_bytes = box_bytes; s.box_rows = box_rows; s.swizzled = swizzled ? 1 : 0;
    s.map = *m;
    s.valid = true;
    return true;
}

template <int FMT, int NT, bool DUAL>
cudaError_t configure_one() {
    cudaError_t e = cudaSuccess;
#define SET_SMEM(V, O)                                                                                                                       \
    if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_stream_kernel<FMT, NT, DUAL, V, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    SET_SMEM(0, false) SET_SMEM(1, false) SET_SMEM(2, false)
    if (NT == 1) { SET_SMEM(0, true) SET_SMEM(1, true) SET_SMEM(2, true) }
#undef SET_SMEM
    return e;
}

// Resident blocks per multiprocessor of the full-featured instantiation at a given dynamic
// shared-memory size (registers can be what limits it), cached per instantiation and size.
template <int FMT, int NT, bool DUAL, bool ONE>
int ext_occupancy(size_t smem) {
    static size_t at_smem = 0;
    static int blocks = -1;
    if (blocks < 0 || at_smem != smem) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, linear_stream_kernel<FMT, NT, DUAL, 2, ONE>, THREADS, smem) != cudaSuccess) n = 0;
        blocks = n;
        at_smem = smem;
    }
    return blocks;
}
int ext_blocks_per_sm(int fmt, int nt, bool dual, bool one, size_t smem) {
#define OCC(F)                                                                                         \
    if (fmt == F) {                                                                                    \
        if (nt == 2) return dual ? ext_occupancy<F, 2, true, false>(smem) : ext_occupancy<F, 2, false, false>(smem); \
        if (one) return dual ? ext_occupancy<F, 1, true, true>(smem) : ext_occupancy<F, 1, false, true>(smem);       \
        return dual ? ext_occupancy<F, 1, true, false>(smem) : ext_occupancy<F, 1, false, false>(smem);              \
    }
    OCC(FMT_FP16) OCC(FMT_INT8) OCC(FMT_Q4)
#undef OCC
    return 0;
}

int count_tiles(const LinArgs& a, int tile_rows) {
    if (a.epi == EPI_SWIGLU) return (a.seg[0].N + tile_rows - 1) / tile_rows;
    int n = 0;
    for (int i = 0; i < a.nseg; ++i) n += (a.seg[i].N + tile_rows - 1) / tile_rows;
    return n;
}

}  // namespace

// 2-D byte view of a weight: [rows][rowbytes], box = 128 bytes x box_rows rows, 128-byte swizzle.
bool make_weight_map(CUtensorMap* m, const void* W, int rows, int rowbytes, int box_rows) {
    return cached_byte_map(m, W, rows, rowbytes, 128, box_rows, true);
}

// 2-D byte view of a Q4 scale tensor: [rows][rowbytes], dense box of box_bytes x box_rows.
bool make_scale_map(CUtensorMap* m, const void* S, int rows, int rowbytes, int box_bytes, int box_rows) {
    if (box_bytes % 16 || box_bytes > 256 || box_rows > 256) return false;
    return cached_byte_map(m, S, rows, rowbytes, box_bytes, box_rows, false);
}

bool encode_tiled_2d(void* map, bool half_elems, const void* base, uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes,
                     uint32_t box0, uint32_t box1, bool swizzle128) {
    if (!g_encode_tiled) return false;
    const cuuint64_t dims[2] = {dim0, dim1};
    const cuuint64_t strides[1] = {stride1_bytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1u, 1u};
    return g_encode_tiled(static_cast<CUtensorMap*>(map), half_elems ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                          const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

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
    if ((e = decode_plan_configure()) != cudaSuccess) return e;
    return gemm_tc_configure();
}

// Shapes the streaming kernel takes: 1 <= M <= 16, rows of at least 128 bytes whose
// length is a multiple of 64 bytes (fp16: K % 32, int8: K % 64; Q4: a multiple of 32 bytes,
// K % 64), and 16-byte aligned operands.  Everything else goes to the generic kernel.
bool stream_supported(int fmt, int M, int K, const LinArgs& a) {
    if (M < 1 || M > 16) return false;
    const int rb = fmt_row_bytes(fmt, K);
    // fp16 / int8 consume a row in 64-byte steps; a Q4 step is one 16-byte block, and its scale
    // rows are copied in 4-byte pieces (two blocks), so Q4 rows only have to be whole pairs of blocks
    if (rb < 128 || (rb % (fmt == FMT_Q4 ? 32 : 64)) != 0) return false;
    // int8: the limb sums are 32-bit; |code| <= 128 times a limb <= 255 over K terms must stay below 2^31
    if (fmt == FMT_INT8 && K > 65536) return false;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    for (int i = 0; i < a.nseg; ++i) {
        if (!al16(a.seg[i].W)) return false;
        if (fmt == FMT_Q4 && (reinterpret_cast<uintptr_t>(a.seg[i].scale) & 3)) return false;
    }
    if (a.epi == EPI_SWIGLU && (!al16(a.W2) || (fmt == FMT_Q4 && (reinterpret_cast<uintptr_t>(a.scale2) & 3)))) return false;
    if (!al16(a.x)) return false;
    if (a.norm_w && !al16(a.norm_w)) return false;
    return true;
}

// Geometry heuristics:
//   * many rows: each consumer warp owns 32 rows of a 128-row block tile, stages are
//     256 bytes of every row;
//   * few rows: the four consumers split K of a 32-row tile so that the whole operator is
//     requested at once;
//   * the grid is sized so that every block gets the same number of tiles.
StreamPlan stream_plan(int fmt, const LinArgs& a, int sm_count, size_t smem_limit) {
    StreamPlan p = {};
    const int M = a.M, K = a.K;
    const bool dual = a.epi == EPI_SWIGLU, norm = a.norm_w != nullptr;
    const int rb = fmt_row_bytes(fmt, K);
    const int nt = M > 8 ? 2 : 1;
    const int rb_cols = ((rb + 127) / 128) * 128;
    const int warp_rows = dual ? 16 : WARP_ROWS;
    int kw = count_tiles(a, NCW * warp_rows) < 2 * sm_count && rb_cols >= 256 ? NCW : 1;
    if (kw != 1 && fmt == FMT_Q4 && a.sk_scratch && a.sk_flags) {
        // Between one and two 128-row tiles per SM with long rows (28672 x 8192: 224 tiles of 16 chunks): whole-row
        // tiles dealt out evenly as pipeline items (the balanced launch below) beat the K split, which pays a
        // four-way reduction and an epilogue per 32 rows (measured 33.8 against 37.6 us); with fewer than eight
        // items per block the balanced launch does not apply and the K split stays (24576 x 4096: 16.6 against 19.6 us)
        const int t128 = count_tiles(a, NCW * warp_rows);
        const long long items = (long long)t128 * ((rb + 255) / 256);
        if (t128 > sm_count && items >= (long long)8 * 2 * sm_count) kw = 1;
    }
    int kcb = 256;
    if (kw != 1) {
        kcb = (((rb + NCW - 1) / NCW + 127) / 128) * 128;  // one chunk per consumer when the row is short
        if (kcb > 384) kcb = 256;
    }
    if (kcb > rb_cols) kcb = rb_cols;
    while ((size_t)make_geo(fmt, M, K, kcb, 2, nt, norm).total > smem_limit && kcb > 128) kcb -= 128;
    if ((size_t)make_geo(fmt, M, K, kcb, 2, nt, norm).total > smem_limit) { p.ok = false; return p; }
    const int ntiles = count_tiles(a, kw == 1 ? NCW * warp_rows : warp_rows);
    const int nchunks = (rb + kcb - 1) / kcb;
    const int groups = kw == 1 ? nchunks : (nchunks + NCW - 1) / NCW;
    // Ring depth and blocks per SM (measured on B200): two blocks per SM with a three-stage
    // ring stream long operators best; a block with only a few pipeline items gets a ring as
    // deep as its item count, so that the whole operator is in flight after the first request.
    int per_sm = 0;
    for (int ps = 2; ps >= 1 && !per_sm; --ps) {
        const size_t budget = (smem_limit + 1024) / ps - 1024;
        int st = ps >= 2 ? 4 : 6;
        while (st > 2 && (size_t)make_geo(fmt, M, K, kcb, st, nt, norm).total > budget) --st;
        if ((size_t)make_geo(fmt, M, K, kcb, st, nt, norm).total > budget) continue;
        const int resident = sm_count * ps;
        const int items = ((ntiles + resident - 1) / resident) * groups;  // pipeline items of the busiest block
        if (items <= st) st = items < 2 ? 2 : items;
        else if (st > 3) st = 3;
        per_sm = ps;
        p.stages = st;
    }
    if (per_sm == 0) { p.ok = false; return p; }
    const int stages = p.stages;
    Geo g = make_geo(fmt, M, K, kcb, stages, nt, norm);
    const int resident = sm_count * per_sm;
    const int waves = (ntiles + resident - 1) / resident;
    p.grid = waves > 0 ? (ntiles + waves - 1) / waves : 1;
    if (p.grid < 1) p.grid = 1;
    // Whole tiles leave SMs idle when the tile count is an awkward multiple of the SM count
    // (224 tiles on 148 SMs: some SMs run two blocks, some one).  For operators large enough
    // that the fix-up's latency does not matter, deal the items out evenly instead.
    {
        size_t wbytes = 0;
        for (int i = 0; i < a.nseg; ++i) wbytes += (size_t)a.seg[i].N * rb;
        const int sm_blocks = (p.grid + sm_count - 1) / sm_count;
        const double plain_eff = (double)ntiles / ((double)sm_count * sm_blocks * (waves > 0 ? waves : 1));
        const long long total = (long long)ntiles * groups;
        const long long per_block = (total + resident - 1) / resident;
        const double sk_eff = (double)total / ((double)resident * (double)per_block);
        // (measured: it pays for the instruction-bound Q4 kernel with long rows; the int8 and fp16
        // kernels are HBM-bound, idle SM slots cost them nothing and the fix-up only adds latency)
        const int want = (fmt == FMT_Q4 && wbytes >= ((size_t)8 << 20) && plain_eff < 0.9 && sk_eff > plain_eff + 0.05 && per_block >= 8) ? 1 : 0;
        // blocks that share a tile wait on one another: all of them must be resident at once
        if (want && a.sk_scratch && a.sk_flags && resident <= SK_MAX_BLOCKS && total >= resident &&
            ext_blocks_per_sm(fmt, nt, dual, M == 1 && nt == 1, (size_t)g.total) >= per_sm) {
            p.streamk = true;
            p.grid = resident;
        }
    }
    p.kcb = kcb;
    p.kw = kw;
    p.warps = NCW;
    p.ntiles = ntiles;
    p.smem = (size_t)g.total;
    p.ok = true;
    return p;
}

cudaError_t launch_stream(int fmt, const LinArgs& a, const StreamPlan& p, cudaStream_t st, bool pdl) {
    KArgsQ4 ka;  // sliced to KArgs for the formats without block scales
    ka.a = a;
    ka.a.kcb = p.kcb;
    ka.a.kw = p.kw;
    ka.a.ntiles = p.ntiles;
    ka.a.streamk = p.streamk ? 1 : 0;
    ka.stages = p.stages;
    ka.rowbytes = fmt_row_bytes(fmt, a.K);
    ka.nchunks = (ka.rowbytes + p.kcb - 1) / p.kcb;
    size_t wbytes = 0;
    for (int i = 0; i < a.nseg; ++i) wbytes += (size_t)a.seg[i].N * ka.rowbytes;
    ka.evict_first = wbytes > ((size_t)96 << 20) ? 1 : 0;  // weights that cannot stay in L2 anyway are streamed evict-first
    const bool dual = a.epi == EPI_SWIGLU;
    const int nt = a.M > 8 ? 2 : 1;
    const int warp_rows = dual ? 16 : WARP_ROWS;
    const int tile_rows = p.kw == 1 ? NCW * warp_rows : warp_rows;
    int t0 = 0;
    for (int i = 0; i < a.nseg; ++i) {
        ka.a.seg[i].tile0 = t0;
        t0 += (a.seg[i].N + tile_rows - 1) / tile_rows;
        if (!make_weight_map(&ka.tm[i], a.seg[i].W, a.seg[i].N, ka.rowbytes, tile_rows)) return cudaErrorInvalidValue;
    }
    if (dual && !make_weight_map(&ka.tm[3], a.W2, a.seg[0].N, ka.rowbytes, tile_rows)) return cudaErrorInvalidValue;
    // Q4 block scales by tensor copy: the scale rows (K / 16 bytes each) must keep 16-byte
    // pitch and alignment; otherwise the consumers fetch them with cp.async
    ka.scale_tma = 0;
    const uint16_t* sbase[4];
    int srow = 0;
    if (fmt == FMT_Q4 && q4_scale_views(a, sbase, &srow)) {
        bool ok = true;
        const int bw = p.kcb / 8;
        for (int i = 0; ok && i < a.nseg; ++i) ok = make_scale_map(&ka.tm_s[i], sbase[i], a.seg[i].N, srow, bw, tile_rows);
        if (ok && dual) ok = make_scale_map(&ka.tm_s[3], sbase[3], a.seg[0].N, srow, bw, tile_rows);
        ka.scale_tma = ok ? 1 : 0;
    }
#define GO(F)                                                                                                  \
    if (fmt == F) {                                                                                            \
        if (dual) return nt == 2 ? launch_t<F, 2, true>(ka, p, st, pdl) : launch_t<F, 1, true>(ka, p, st, pdl); \
        return nt == 2 ? launch_t<F, 2, false>(ka, p, st, pdl) : launch_t<F, 1, false>(ka, p, st, pdl);         \
    }
    GO(FMT_FP16) GO(FMT_INT8) GO(FMT_Q4)
#undef GO
    return cudaErrorInvalidValue;
}


}  // namespace nnb
