// Resident decode step, sm_100a: one launch runs a whole run of recorded single-token operators.
//
// Stands in for the reference's recordable-queue replay of a decode step
// (src/models/smollm2-135m-instruct/src/model.cpp:104-195,312-344; src/models/lfm2-5-350m/src/
// model.cpp:188-228,376-458), whose purpose is to remove the per-dispatch cost between the
// M == 1 GEMVs of a token.  A CUDA graph of separate launches still pays about a microsecond of
// dependent-launch latency plus the kernel prologue per operator, ten times the HBM time of a
// 0.3-1.8 MB per-layer weight.  Here the blocks stay resident and walk a table of operator
// descriptors (plan.h):
//
//   * tile j of the run (tiles are numbered through all operators) belongs to block j mod G, so
//     every block holds about the same number of tiles and knows them without any communication;
//   * the producer warp's elected lane streams the block's tiles, operator after operator, into a
//     byte ring of shared memory with tiled tensor copies (cp.async.bulk.tensor, 128-byte swizzle,
//     the descriptors' tensor maps read in place from global memory).  Weights never depend on
//     activations, so the producer runs as far ahead as the ring allows: the weights of the next
//     operators, often of the next layers, are already in shared memory when their activations
//     arrive.  Items have the operator's own size; a table of PLAN_SLOTS mbarrier pairs tracks them;
//   * activations go from one operator to the next through device memory, each 8-byte word carrying
//     two fp16 values and the epoch of the operator that produced them.  A reader polls the words
//     until they show the epoch it expects: the word is its own arrival mark, so there is no fence,
//     no counter and no grid-wide barrier on the path, and an operator starts as soon as its own
//     inputs exist.  Which operator produces which input, which stores are overwritten later in the
//     run and which hazards the data flow itself orders is worked out when the run is recorded
//     (plan.cpp: analyze_run);
//   * the arithmetic is the separate launch's (stream_core.cuh), on the same K partition and in the
//     same order, so a run gives the same bits as the operators launched one by one.  A per-layer
//     operator is bound by latency, not by its weight stream, so a block has eight consumer warps: a
//     tile whose K is split has sixteen K parts and every warp takes two of them; int8 weights of such
//     tiles are multiplied with the fp16 activations as they are (no fixed-point copy to build once the
//     activations arrive).  What does not depend on the activations (descriptor, norm weight, row
//     scales, the values an in-place epilogue updates, the tile's weights) is fetched or waited for
//     before the wait for them, so that little is left to do once they are there;
//   * every wait (ring slot, weights, activations) is bounded; when one runs out the block records
//     the status, raises the run's abort flag so that the other blocks stop waiting too, keeps
//     walking its items so that its barriers and copies complete, and returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "plan.h"
#include "ptx.cuh"
#include "stream_core.cuh"

namespace nnb {

namespace {

__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// The descriptors' tensor maps sit in global memory and were written by the host (cudaMemcpy when
// the run was built): the thread that hands one to the TMA unit first orders its view of those 128
// bytes behind the host's writes, in the tensor-map proxy.
__device__ __forceinline__ void tensormap_acquire(const void* tmap) {
    asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(tmap) : "memory");
}

// First tile of an operator that belongs to block b: tile j sits on block (tile_start + j) mod G.
__device__ __forceinline__ int first_tile(int tile_start_mod, int b, int G) {
    const int f = b - tile_start_mod;
    return f < 0 ? f + G : f;
}

// Placement of the next ring item: items are laid out one after another and start over at the
// ring's head when they would run past its end.  Producer and consumers compute it alike.
__device__ __forceinline__ int ring_place(int& head, int bytes, int ring_bytes) {
    if (head + bytes > ring_bytes) head = 0;
    const int off = head;
    head += bytes;
    return off;
}

constexpr int PCW = KPARTS;               // consumer warps of the resident kernel: one per K part of a split tile
constexpr int PTHREADS = PCW * 32;        // consumer threads
constexpr int PLAN_BLOCK = PTHREADS + 32; // + the producer warp
static_assert(PLAN_BLOCK == DECODE_PLAN_THREADS, "block size");

__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(PTHREADS) : "memory"); }

struct CState {            // consumer-side state carried from operator to operator (the same in every consumer thread;
                           // kept in shared memory between operators, in registers inside one)
    int head;              // ring placement
    unsigned n;            // items consumed so far
    int ti;                // tiles finished so far (selects the reduction buffer)
    bool failed;
    unsigned ebase;        // epoch of operator i of this launch = ebase + i + 1
    // what the staged activations in shared memory currently hold
    const void* st_src;
    unsigned st_epoch;
    int st_fmt;
    const void* st_norm;
    const void* st_gamma;  // the norm weight held in shared memory
    uint32_t st_xrow;      // shared-memory address of the staged activations
};

__device__ __noinline__ void report_failure(int* status, unsigned* state, int code) {
    *reinterpret_cast<volatile int*>(status) = code;
    atomicExch(state + 2, 1u);
}
__device__ __forceinline__ void record_failure(const PlanParams& P, CState& S, int code) {
    S.failed = true;
    report_failure(P.status, P.state, code);
}
// The slow part of a wait for a ring item: out of line, since it is taken only when the weights are late.
__device__ __noinline__ bool wait_full_slow(uint32_t bar, uint32_t parity, long long limit) { return mbar_wait_bounded(bar, parity, limit); }

// Poll published words until each carries `epoch`, and leave their fp16 pairs in dst.  Thread tid
// takes words base + tid + j * PTHREADS, j < B; all of a thread's loads are in flight together, and a
// word is asked for again only while it has not arrived.
template <int B>
__device__ __forceinline__ void poll_batch(const PlanParams& P, CState& S, const unsigned long long* ll, int base, int nw, unsigned epoch,
                                           uint32_t* dst, int tid) {
    unsigned long long w[B];
    unsigned pending = 0u;
#pragma unroll
    for (int j = 0; j < B; ++j) {
        w[j] = 0ull;
        if (base + j * PTHREADS + tid < nw) pending |= 1u << j;
    }
    const long long t0 = clock64();
    unsigned spins = 0;
    while (pending) {
#pragma unroll
        for (int j = 0; j < B; ++j)
            if (pending & (1u << j)) w[j] = ld_relaxed_u64(ll + base + j * PTHREADS + tid);
#pragma unroll
        for (int j = 0; j < B; ++j)
            if ((unsigned)(w[j] >> 32) == epoch) pending &= ~(1u << j);
        if (pending) {
            if (S.failed) break;  // an earlier wait of this launch ran out: take what is there
            if ((++spins & 31u) == 0u) {
                if (clock64() - t0 > P.wait_cycles) {
                    record_failure(P, S, 4);
                    break;
                }
                if (ld_relaxed_u32(P.state + 2)) {  // another block gave up: do not wait either
                    S.failed = true;
                    break;
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < B; ++j) {
        const int idx = base + j * PTHREADS + tid;
        if (idx < nw) dst[idx] = (uint32_t)w[j];
    }
}
__device__ __forceinline__ void poll_words(const PlanParams& P, CState& S, const unsigned long long* ll, int nw, unsigned epoch, uint32_t* dst,
                                           int tid) {
    if (nw <= PTHREADS) {
        poll_batch<1>(P, S, ll, 0, nw, epoch, dst, tid);
    } else if (nw <= 2 * PTHREADS) {
        poll_batch<2>(P, S, ll, 0, nw, epoch, dst, tid);
    } else {
        for (int base = 0; base < nw; base += 4 * PTHREADS) poll_batch<4>(P, S, ll, base, nw, epoch, dst, tid);
    }
}

// RMSNorm of the single row x (in shared or global memory) with the norm weight gw (in shared
// memory): xn[k] = half((x[k] * rsqrt(mean x^2 + eps)) * gw[k]).  Run by the first NCW consumer warps
// (barrier 2), with the sums taken in the order of rmsnorm_rows (stream_core.cuh) so that both give
// the same bits.
__device__ __forceinline__ void rmsnorm_row_smem(const uint16_t* x, const uint16_t* gw, float n_eps, int aK, uint16_t* xn, float* red, int tid,
                                                 int lane, int warp) {
    const int per_row = aK / 8;
    float ss = 0.f;
    for (int p = tid; p < per_row; p += NCW * 32) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + p * 8);
        const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wv[q]));
            ss += f.x * f.x;
            ss += f.y * f.y;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp * 16] = ss;
    asm volatile("bar.sync 2, %0;" ::"n"(NCW * 32) : "memory");
    float tot = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < NCW; ++w2) tot += red[w2 * 16];
    const float inv = 1.0f / sqrtf(tot / (float)aK + n_eps);
    for (int p = tid; p < per_row; p += NCW * 32) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + p * 8);
        const uint4 g4 = *reinterpret_cast<const uint4*>(gw + p * 8);
        const uint32_t xv[4] = {v.x, v.y, v.z, v.w}, gv[4] = {g4.x, g4.y, g4.z, g4.w};
        uint32_t o4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 fx = __half22float2(*reinterpret_cast<const __half2*>(&xv[q]));
            const float2 fg = __half22float2(*reinterpret_cast<const __half2*>(&gv[q]));
            const __half2 h = __floats2half2_rn((fx.x * inv) * fg.x, (fx.y * inv) * fg.y);
            o4[q] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(xn + p * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
    }
}

// The fp16 value of row n from the published copy (in-place epilogues).  `w` is the word as it was
// fetched ahead of time; it is polled again only if it did not carry the epoch yet.
__device__ __forceinline__ uint16_t poll_row(const PlanParams& P, CState& S, const unsigned long long* ll, int n, unsigned epoch,
                                             unsigned long long w) {
    const unsigned long long* p = ll + (n >> 1);
    if ((unsigned)(w >> 32) != epoch && !S.failed) {
        const long long t0 = clock64();
        unsigned spins = 0;
        for (;;) {
            w = ld_relaxed_u64(p);
            if ((unsigned)(w >> 32) == epoch) break;
            if ((++spins & 31u) == 0u) {
                if (clock64() - t0 > P.wait_cycles) {
                    record_failure(P, S, 5);
                    break;
                }
                if (ld_relaxed_u32(P.state + 2)) {
                    S.failed = true;
                    break;
                }
            }
        }
    }
    return (uint16_t)((n & 1) ? (w >> 16) : w);
}

// One operator on the consumer warps.  D lives in shared memory.
// WIDE: the operator's tiles split K (few rows): eight K parts per tile, one per consumer warp
// (stream_core.cuh: "K parts").  Otherwise the first NCW warps each stream whole rows of a tile,
// exactly as the separate launch does, and the others only keep step with the ring.
// (The two-weight epilogue is a run-time property: the operators of a layer then share one copy of
// the code, which matters because each runs only once per layer and instruction fetch is not free.)
template <int FMT, bool WIDE>
__device__ __noinline__ void run_op(const PlanParams& P, const PlanOpScalars& D, int op, uint8_t* smem, int tid, int lane, int warp) {
    CState S = *reinterpret_cast<const CState*>(smem + PLAN_HDR_STATE);
    const bool DUAL = D.dual != 0;
    const int g = lane >> 2, t = lane & 3;
    const int G = (int)gridDim.x;
    const uint32_t s_base = smem_u32(smem);
    const uint32_t full0 = s_base + PLAN_HDR_BARS, empty0 = full0 + PLAN_SLOTS * 8;
    const int ring_off = (int)(((s_base + (uint32_t)P.off_ring + 1023u) & ~1023u) - s_base);  // tensor copies want 1 KB alignment
    const uint32_t ring = s_base + (uint32_t)ring_off;
    const volatile unsigned* s_issued = reinterpret_cast<const volatile unsigned*>(smem + PLAN_HDR_ISSUED);
    const int aK = D.K, epi = D.epi, kcb = D.kcb, nchunks = D.nchunks, groups = D.groups, rowbytes = D.rowbytes;
    const int item_bytes = D.item_bytes, nbox = D.nbox, ntiles = D.ntiles, nseg = D.nseg;
    const bool scale_tma = (D.flags & PLAN_SCALE_TMA) != 0, row_scales = (D.flags & PLAN_ROW_SCALES) != 0;
    const bool bias_on = (D.flags & PLAN_BIAS) != 0;
    const int scale_off = D.scale_off;
    const int seg1_tile0 = D.seg[1].tile0, seg2_tile0 = D.seg[2].tile0;
    const unsigned epoch = S.ebase + (unsigned)D.epoch;
    const bool publish_ok = op != P.drop_publish_op;
    const int warp_rows = DUAL ? 16 : WARP_ROWS;
    const int tile_rows = WIDE ? warp_rows : NCW * warp_rows;
    const int xstride = x_stride_of(FMT, aK);
    uint8_t* xs = smem + P.off_xs;
    float* red = reinterpret_cast<float*>(smem + P.off_red);

    // WIDE: warp = 2 * quarter + set: chunk `quarter` of every item, units set, set + 2, ... of the chunk
    const int quarter = WIDE ? warp >> 1 : warp, set = warp & 1;
    const bool worker = WIDE || warp < NCW;           // has arithmetic to do
    const int wrow_off = WIDE ? 0 : warp * warp_rows;
    const bool writer = WIDE ? warp == 0 : warp < NCW;  // finishes rows
    auto tile_segment = [&](int tile) {
        int si = 0;
        if (nseg > 1 && tile >= seg1_tile0) si = 1;
        if (nseg > 2 && tile >= seg2_tile0) si = 2;
        return si;
    };
    const int tile_first = first_tile(D.tile_start, (int)blockIdx.x, G);
    const bool inplace = !DUAL && (epi == EPI_RESIDUAL || epi == EPI_SILU_GATE);
    const unsigned res_epoch = S.ebase + (unsigned)D.res_epoch;

    // Everything that does not depend on this operator's activations is requested or done before the
    // wait for them: the previous values of an in-place epilogue (an older operator's output, or memory
    // from before the run) ...
    unsigned long long res_word = 0ull;
    auto fetch_res = [&](int tile) {
        const PlanSeg sg = D.seg[tile_segment(tile)];
        const int n = (tile - sg.tile0) * tile_rows + wrow_off + lane;
        if (writer && inplace && n < sg.N) res_word = D.res_ll ? ld_relaxed_u64(D.res_ll + (n >> 1)) : (unsigned long long)D.res[n];
    };
    if (tile_first < ntiles) fetch_res(tile_first);

    // ... what a tile needs besides its weights and the activations
    constexpr int SETS = WIDE ? 1 : 2;
    constexpr bool IMMA = FMT == FMT_INT8;
    float acc[2][2][1][4];  // WIDE uses set 0 only
    int iacc[IMMA ? 3 : 1][2][1][4];
    unsigned long long am_best = 0ull;
    uint16_t sc1 = 0, res1 = 0;
    PlanSeg sg = D.seg[0];
    int row0 = 0;
    bool scales_ride = false;
    auto tile_prologue = [&](int tile, bool first) {
        sc1 = 0;
        res1 = 0;
        sg = D.seg[DUAL ? 0 : tile_segment(tile)];
        row0 = (tile - sg.tile0) * tile_rows + wrow_off;
        // int8 row scales: with the tile's last item when its rows allow a bulk copy, else from memory now
        scales_ride = FMT == FMT_INT8 && row_scales && plan_rows_bulk_ok(min(tile_rows, sg.N - (tile - sg.tile0) * tile_rows));
        if (writer && FMT == FMT_INT8 && !scales_ride) {
            if (DUAL) {
                const int n = min(row0 + (lane & 15), sg.N - 1);
                sc1 = sg.scale[n];
                res1 = D.scale2[n];  // the up weight's scale rides in the spare register
            } else {
                sc1 = sg.scale[min(row0 + lane, sg.N - 1)];
            }
        }
        if (!first) fetch_res(tile);
#pragma unroll
        for (int u = 0; u < SETS; ++u)
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[u][rb][0][i] = 0.f;
        if (IMMA) {
#pragma unroll
            for (int l = 0; l < 3; ++l)
#pragma unroll
                for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) iacc[l % (IMMA ? 3 : 1)][rb][0][i] = 0;
        }
    };
    if (tile_first < ntiles) tile_prologue(tile_first, true);

    // ... the weights of the block's first item of this operator (normally there already)
    auto claim_item = [&](int& off, unsigned& slot) {
        off = ring_place(S.head, item_bytes, P.ring_bytes);
        slot = S.n % PLAN_SLOTS;
        const unsigned parity = (S.n / PLAN_SLOTS) & 1u;
        ++S.n;
        // A wait that runs out records an error and skips the arithmetic from then on; the warp
        // still walks its items, and still waits for every copy the producer has issued, so that
        // the block's barriers stay matched and nothing is in flight when it returns.
        if (S.n - 1u < *s_issued && !mbar_try_wait(full0 + slot * 8, parity) && !wait_full_slow(full0 + slot * 8, parity, P.wait_cycles)) {
            if (lane == 0 && !S.failed) record_failure(P, S, 1);
            S.failed = true;
        }
        // the lanes of a warp must agree before the warp-wide matrix instructions that follow
        S.failed = __any_sync(0xffffffffu, S.failed) != 0;
    };
    int off_first = 0;
    unsigned slot_first = 0u;
    if (tile_first < ntiles) claim_item(off_first, slot_first);

    // ---------------- activations: fetch (poll the producer's words), normalise, stage ----------------
    // fp16 weights multiply the activations as a plain fp16 row: when the row is in shared memory already
    // (fetched from another operator, or normalised) it is used where it lies and nothing is staged.
    constexpr bool plain = FMT == FMT_FP16;
    constexpr int mode = FMT;
    const void* src_id = D.x_ll ? (const void*)D.x_ll : (const void*)D.x;
    const unsigned x_epoch = D.x_ll ? S.ebase + (unsigned)D.x_epoch : 0u;
    const bool reuse = S.st_src == src_id && S.st_epoch == x_epoch && S.st_fmt == mode && S.st_norm == (const void*)D.norm_w;
    // where the row will be read from is known before it arrives
    const uint32_t x_addr = reuse ? S.st_xrow
                                  : s_base + (uint32_t)(!plain ? P.off_xs : D.norm_w ? P.off_norm : D.x_ll ? P.off_xraw : P.off_xs);
    LaneGeo<1> lg;
    lane_geo_init<FMT, 1>(lg, DUAL, quarter, lane, 1, x_addr, xstride, s_base, smem + P.off_ctab);
    const float* rowscale = reinterpret_cast<const float*>(xs + 3 * xstride + 64);
    if (!reuse) {
        const uint16_t* x_src = D.x;
        // ... and the norm weight, which goes to shared memory
        uint16_t* gamma_s = reinterpret_cast<uint16_t*>(smem + P.off_gamma);
        const bool gamma_fresh = D.norm_w && S.st_gamma != (const void*)D.norm_w;
        if (gamma_fresh) {
            for (int p = tid; p < aK / 8; p += PTHREADS) cp_async_16(smem_u32(gamma_s) + p * 16, D.norm_w + p * 8);
            asm volatile("cp.async.commit_group;" ::: "memory");
            S.st_gamma = (const void*)D.norm_w;
        }
        if (D.x_ll) {
            uint32_t* xraw = reinterpret_cast<uint32_t*>(smem + P.off_xraw);
            poll_words(P, S, D.x_ll, (aK + 1) >> 1, x_epoch, xraw, tid);
            S.failed = __any_sync(0xffffffffu, S.failed) != 0;  // (some lanes may have learnt of a failure, others not)
            x_src = reinterpret_cast<const uint16_t*>(xraw);
        }
        if (IMMA && tid < 16) reinterpret_cast<uint32_t*>(xs + 3 * xstride)[tid] = 0u;  // the row-maximum words
        if (gamma_fresh) asm volatile("cp.async.wait_group 0;" ::: "memory");
        // everyone is done with the previous staging and reduction buffers; the fetched row is complete
        consumers_sync();
        if (D.norm_w) {
            uint16_t* xn = reinterpret_cast<uint16_t*>(smem + P.off_norm);
            if (warp < NCW) rmsnorm_row_smem(x_src, gamma_s, D.norm_eps, aK, xn, red, tid, lane, warp);
            consumers_sync();
            x_src = xn;
        }
        if (plain) {
            if (!D.x_ll && !D.norm_w) {  // a row in global memory: bring it in
                stage_x<FMT_FP16>(x_src, 1, aK, xs, aK * 2 + 16, nullptr, tid, PTHREADS);
                consumers_sync();
            }
        } else {
            if (IMMA) stage_x_int8(x_src, 1, aK, xs, xstride, tid, PTHREADS);
            else stage_x<FMT>(x_src, 1, aK, xs, xstride, reinterpret_cast<float*>(smem + P.off_ctab), tid, PTHREADS);
            consumers_sync();
        }
        S.st_xrow = x_addr;
        S.st_src = src_id;
        S.st_epoch = x_epoch;
        S.st_fmt = mode;
        S.st_norm = (const void*)D.norm_w;
    }

    for (int tile = tile_first; tile < ntiles;) {
        // ---- the tile's pipeline items ----
        for (int cg = 0; cg < groups; ++cg) {
            const int c = WIDE ? cg * NCW + quarter : cg;
            const bool active = worker && c < nchunks;
            int off = off_first;
            unsigned slot = slot_first;
            if (tile != tile_first || cg != 0) claim_item(off, slot);
            const uint32_t sw = ring + (uint32_t)off;
            const int cb = (S.failed || !active) ? 0 : min(kcb, rowbytes - c * kcb);
            if (FMT == FMT_INT8 && scales_ride && writer && cg == groups - 1) {
                const uint16_t* sc = reinterpret_cast<const uint16_t*>(smem + ring_off + off + scale_off);
                if (DUAL) {
                    sc1 = sc[wrow_off + (lane & 15)];
                    res1 = sc[256 + wrow_off + (lane & 15)];
                } else {
                    sc1 = sc[wrow_off + lane];
                }
            }
            if constexpr (FMT == FMT_FP16) {
                if constexpr (WIDE) {
                    const int s0 = (c * kcb) / 64;
                    for (int u = set; u < cb / 64; u += 2) step_fp16<1>(lg, sw, s0 + u, u, acc[0]);
                } else {
                    chunk_fp16<1>(lg, sw, c, kcb, cb, acc);
                }
            } else if constexpr (FMT == FMT_INT8) {
                if constexpr (WIDE) {
                    const int s0 = (c * kcb) / 64;
                    for (int u = set; u < cb / 64; u += 2) step_int8<1>(lg, sw, s0 + u, u, iacc);
                } else {
                    chunk_int8<1>(lg, sw, c, kcb, cb, iacc);
                }
            } else {
                // block scales arrive by tensor copies: whole boxes, which for two weights means all
                // gate rows first, then all up rows
                const int sstr = scale_tma ? kcb / 8 : stage_sstride(kcb);
                const int srow0 = (scale_tma && DUAL) ? quarter * (WARP_ROWS / 2) : quarter * WARP_ROWS;
                const int srow1 = (scale_tma && DUAL) ? NCW * WARP_ROWS / 2 + quarter * (WARP_ROWS / 2) : quarter * WARP_ROWS + 16;
                const uint8_t* scb = smem + ring_off + off + nbox * CTA_BOX;
                const uint8_t* const sc_rb[2] = {scb + (srow0 + g) * sstr, scb + (srow1 + g) * sstr};
                if constexpr (WIDE) {
                    for (int u = set; u < cb / 16; u += 2) block_q4_at<1>(lg, sw, c, kcb, u, acc[0], sc_rb, sstr);
                } else {
                    chunk_q4<1>(lg, sw, c, kcb, cb, acc, sc_rb, sstr);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + slot * 8);  // hand the item's bytes back to the producer
        }
        ++S.ti;

        // ---- tile finished.  The token's results sit in the lanes with t == 0: rows g and g + 8 of each
        //      row block.  Row L of the tile is finished by lane L of the warp that holds its sum. ----
        float v0, v1 = 0.f;  // v1: the second weight's sum (two-weight epilogue)
        if constexpr (WIDE) {
            // The eight K parts meet in shared memory.  Per consumer of the separate launch (quarter) the
            // two sets are added first, then the quarters in order; int8 parts are exact integer limb
            // sums, added as integers and turned into a float once per quarter, as that consumer does.
            const int r0 = DUAL ? (lane & 15) : lane;
            if constexpr (IMMA) {
                int* ibuf = reinterpret_cast<int*>(red) + (S.ti & 1) * (KPARTS * 3 * 32);
                if (t == 0) {
#pragma unroll
                    for (int l = 0; l < 3; ++l) {
                        int* mine = ibuf + (warp * 3 + l) * 32 + g;
                        mine[0] = iacc[l][0][0][0];
                        mine[8] = iacc[l][0][0][2];
                        mine[16] = iacc[l][1][0][0];
                        mine[24] = iacc[l][1][0][2];
                    }
                }
                consumers_sync();
                auto quarter_sum = [&](int q, int r) {
                    const int* a = ibuf + (2 * q) * 3 * 32 + r;
                    const int* b2 = a + 3 * 32;
                    const float f = fmaf((float)(a[0] + b2[0]), 65536.f, fmaf((float)(a[32] + b2[32]), 256.f, (float)(a[64] + b2[64])));
                    return f * rowscale[0] + 0.f;  // (+ 0: the consumer adds its empty second set)
                };
                v0 = quarter_sum(0, r0);
#pragma unroll
                for (int q = 1; q < NCW; ++q) v0 += quarter_sum(q, r0);
                if (DUAL) {
                    v1 = quarter_sum(0, 16 + r0);
#pragma unroll
                    for (int q = 1; q < NCW; ++q) v1 += quarter_sum(q, 16 + r0);
                }
            } else {
                float* buf = red + (S.ti & 1) * (KPARTS * 32);
                if (t == 0) {
                    float* mine = buf + warp * 32 + g;
                    mine[0] = acc[0][0][0][0];
                    mine[8] = acc[0][0][0][2];
                    mine[16] = acc[0][1][0][0];
                    mine[24] = acc[0][1][0][2];
                }
                consumers_sync();
                v0 = buf[r0] + buf[32 + r0];
#pragma unroll
                for (int q = 1; q < NCW; ++q) v0 += buf[(2 * q) * 32 + r0] + buf[(2 * q + 1) * 32 + r0];
                if (DUAL) {
                    v1 = buf[16 + r0] + buf[32 + 16 + r0];
#pragma unroll
                    for (int q = 1; q < NCW; ++q) v1 += buf[(2 * q) * 32 + 16 + r0] + buf[(2 * q + 1) * 32 + 16 + r0];
                }
            }
        } else {
            if constexpr (IMMA) int8_recombine<1>(iacc, acc[0], rowscale, 1, t);
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[0][rb][0][i] += acc[1][rb][0][i];
            const int src = (lane & 7) * 4;
            const float a00 = __shfl_sync(0xffffffffu, acc[0][0][0][0], src), a02 = __shfl_sync(0xffffffffu, acc[0][0][0][2], src);
            const float a10 = __shfl_sync(0xffffffffu, acc[0][1][0][0], src), a12 = __shfl_sync(0xffffffffu, acc[0][1][0][2], src);
            if (DUAL) {
                const int hi = (lane >> 3) & 1;
                v0 = hi ? a02 : a00;
                v1 = hi ? a12 : a10;
            } else {
                const int sel = lane >> 3;
                v0 = sel == 0 ? a00 : sel == 1 ? a02 : sel == 2 ? a10 : a12;
            }
        }

        // ---- epilogue (the warp that holds the tile's sums) ----
        uint16_t hv = 0;
        const int n = row0 + lane;
        const bool valid = writer && (DUAL ? lane < 16 : true) && n < sg.N;
        if (valid) {
            if (DUAL) {
                hv = finish_swiglu<FMT>(v0, v1, sc1, res1);
            } else {
                if (inplace) res1 = D.res_ll ? poll_row(P, S, D.res_ll, n, res_epoch, res_word) : (uint16_t)res_word;
                hv = finish_row<FMT>(v0, sc1, epi, res1);
                if (bias_on) {
                    // the reference adds the bias to the stored fp16 result, in fp32, and rounds again
                    const uint16_t* bp = P.bias[op * 3 + tile_segment(tile)];
                    if (bp) hv = __half_as_ushort(__float2half_rn(__fadd_rn(__half2float(__ushort_as_half(hv)), __half2float(__ushort_as_half(bp[n])))));
                }
            }
        }
        if (valid && sg.out) sg.out[n] = hv;
        if (sg.ll_out && writer) {
            // two rows and the epoch in one 8-byte word: the word is its own arrival mark
            const unsigned other = __shfl_down_sync(0xffffffffu, (unsigned)hv, 1);
            if (valid && !(lane & 1) && publish_ok) {
                const unsigned pair = (unsigned)hv | ((n + 1 < sg.N) ? other << 16 : 0u);
                st_relaxed_u64(sg.ll_out + (n >> 1), ((unsigned long long)epoch << 32) | pair);
            }
        }
        if (D.argmax_slot && valid && (hv & 0x7FFFu) <= 0x7C00u) {  // NaNs never win
            const unsigned long long key = argmax_key_half(hv, D.argmax_base + n);
            am_best = key > am_best ? key : am_best;
        }
        tile += G;
        if (tile < ntiles) tile_prologue(tile, false);
    }

    if (D.argmax_slot) {
        // fused greedy pick: one atomic per warp, then the last block of this operator publishes the index
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, am_best, o);
            am_best = other > am_best ? other : am_best;
        }
        if (lane == 0 && am_best) atomicMax(D.argmax_slot, am_best);
        __threadfence();
        consumers_sync();
        if (tid == 0) {
            const unsigned prev = atomicAdd(D.argmax_done, 1u);
            if (prev == (unsigned)D.nblocks - 1u) {
                __threadfence();
                const unsigned long long k = *reinterpret_cast<volatile unsigned long long*>(D.argmax_slot);
                *reinterpret_cast<volatile unsigned long long*>(D.argmax_slot) = 0ull;
                *reinterpret_cast<volatile unsigned*>(D.argmax_done) = 0u;
                *D.argmax_out = k ? (int)(0xFFFFFFFFu - (unsigned int)(k & 0xFFFFFFFFull)) : -1;
            }
        }
    }
    // (the next operator reads the state after the consumers' barrier at its start)
    if (tid == 0) *reinterpret_cast<CState*>(smem + PLAN_HDR_STATE) = S;
}

__global__ void __launch_bounds__(PLAN_BLOCK, 1) decode_plan_kernel(const __grid_constant__ PlanParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = (int)gridDim.x, b = (int)blockIdx.x;
    const uint32_t s_base = smem_u32(smem);
    const uint32_t full0 = s_base + PLAN_HDR_BARS, empty0 = full0 + PLAN_SLOTS * 8;
    int* slot_off = reinterpret_cast<int*>(smem + PLAN_HDR_SLOTS);  // producer's record of the items in flight
    int* slot_end = slot_off + PLAN_SLOTS;
    volatile unsigned* s_issued = reinterpret_cast<volatile unsigned*>(smem + PLAN_HDR_ISSUED);  // items the producer has issued, once it stops early
    int2* s_tiles = reinterpret_cast<int2*>(smem + P.off_tiles);
    const int nops = P.nops;
    const int ring_off = (int)(((s_base + (uint32_t)P.off_ring + 1023u) & ~1023u) - s_base);

    if (tid < 16) reinterpret_cast<uint32_t*>(smem)[tid] = 0u;  // 64 bytes of zeros: B operand of absent token rows
    if (tid == 0) {
        *s_issued = 0xFFFFFFFFu;
        for (int s = 0; s < PLAN_SLOTS; ++s) {
            mbar_init(full0 + s * 8, 1u);
            mbar_init(empty0 + s * 8, (uint32_t)PCW);
        }
        mbar_init_fence();
    }
    for (int i = tid; i < nops; i += PLAN_BLOCK) s_tiles[i] = P.op_tiles[i];  // written before the launch, never by it
    __syncthreads();

    // ================= producer warp: one elected lane feeds the TMA unit =================
    if (warp == PCW) {
        pdl_launch_dependents();
        if (lane != 0) return;
        int head = 0;
        unsigned n = 0, oldest = 0;
        for (int op = 0; op < nops; ++op) {
            const int2 tt = s_tiles[op];
            int tile = first_tile(tt.x, b, G);
            if (tile >= tt.y) continue;
            const PlanOp* D = P.ops + op;
            const int fmt = __ldg(&D->s.fmt), dual = __ldg(&D->s.dual), ksplit = __ldg(&D->s.ksplit), kcb = __ldg(&D->s.kcb);
            const int nchunks = __ldg(&D->s.nchunks), groups = __ldg(&D->s.groups), rowbytes = __ldg(&D->s.rowbytes), nseg = __ldg(&D->s.nseg);
            const int item_bytes = __ldg(&D->s.item_bytes), nbox = __ldg(&D->s.nbox);
            const int flags = __ldg(&D->s.flags), scale_off = __ldg(&D->s.scale_off);
            const bool stma = fmt == FMT_Q4 && (flags & PLAN_SCALE_TMA) != 0;
            const bool row_scales = (flags & PLAN_ROW_SCALES) != 0;
            auto ldg_ptr = [](const uint16_t* const* pp) { return reinterpret_cast<const uint16_t*>(__ldg(reinterpret_cast<const unsigned long long*>(pp))); };
            const int seg1_tile0 = __ldg(&D->s.seg[1].tile0), seg2_tile0 = __ldg(&D->s.seg[2].tile0);
            const uint64_t policy = (flags & PLAN_EVICT_FIRST) ? l2_policy_evict_first() : l2_policy_evict_normal();
            const int warp_rows = dual ? 16 : WARP_ROWS;
            const int tile_rows = ksplit ? warp_rows : NCW * warp_rows;
            const int bw = kcb / 8;  // bytes of block scales per row and item
            for (int k = 0; k < (dual ? 1 : nseg); ++k) {
                tensormap_acquire(&D->tm[k]);
                if (stma) tensormap_acquire(&D->tm_s[k]);
            }
            if (dual) {
                tensormap_acquire(&D->tm[3]);
                if (stma) tensormap_acquire(&D->tm_s[3]);
            }
            for (; tile < tt.y; tile += G) {
                int sg = 0, sg_tile0 = 0;
                if (!dual) {
                    if (nseg > 1 && tile >= seg1_tile0) { sg = 1; sg_tile0 = seg1_tile0; }
                    if (nseg > 2 && tile >= seg2_tile0) { sg = 2; sg_tile0 = seg2_tile0; }
                }
                const int row0 = (tile - sg_tile0) * tile_rows;
                const int rows_valid = row_scales ? min(tile_rows, __ldg(&D->s.seg[sg].N) - row0) : 0;
                const bool scales_ride = row_scales && plan_rows_bulk_ok(rows_valid);
                for (int cg = 0; cg < groups; ++cg) {
                    // the tile's row scales travel with its last item
                    const uint32_t sc_bytes = (scales_ride && cg == groups - 1) ? (uint32_t)rows_valid * 2u : 0u;
                    const int off = ring_place(head, item_bytes, P.ring_bytes);
                    // The bytes must be free.  Items leave the ring in the order they entered it, so the
                    // youngest item in flight that overlaps the new one decides how far to wait (the
                    // table may still list older items that were released long ago, in other places).
                    unsigned need = oldest;
                    for (unsigned j = oldest; j != n; ++j) {
                        const unsigned js = j % PLAN_SLOTS;
                        if (max(off, slot_off[js]) < min(off + item_bytes, slot_end[js])) need = j + 1u;
                    }
                    if (n - oldest == (unsigned)PLAN_SLOTS && need == oldest) need = oldest + 1u;  // the new item's own slot
                    while (oldest != need) {
                        // (four times the consumers' limit: a consumer that gives up on its own wait
                        // releases its items right after, and the producer should still be there)
                        if (!mbar_wait_bounded(empty0 + (oldest % PLAN_SLOTS) * 8, (oldest / PLAN_SLOTS) & 1u, 4 * P.wait_cycles)) {
                            *reinterpret_cast<volatile int*>(P.status) = 2;
                            atomicExch(P.state + 2, 1u);
                            *s_issued = n;
                            return;
                        }
                        ++oldest;
                    }
                    const unsigned slot = n % PLAN_SLOTS;
                    slot_off[slot] = off;
                    slot_end[slot] = off + item_bytes;
                    ++n;
                    const uint32_t dst = s_base + (uint32_t)(ring_off + off), bar = full0 + slot * 8;
                    auto send_row_scales = [&]() {
                        if (!sc_bytes) return;
                        bulk_g2s(dst + scale_off, ldg_ptr(&D->s.seg[sg].scale) + row0, sc_bytes, bar, policy);
                        if (dual) bulk_g2s(dst + scale_off + 512, ldg_ptr(&D->s.scale2) + row0, sc_bytes, bar, policy);
                    };
                    if (!ksplit) {
                        // one copy per 128-byte column covers the rows of all four consumers
                        const int cb = min(kcb, rowbytes - cg * kcb);
                        const int nb = (cb + 127) >> 7;
                        mbar_arrive_expect_tx(bar, (uint32_t)(nb * CTA_BOX + (stma ? NCW * WARP_ROWS * bw : 0)) + (dual ? 2u : 1u) * sc_bytes);
                        send_row_scales();
                        if (stma) {
                            const uint32_t sdst = dst + nbox * CTA_BOX;
                            if (dual) {
                                tma_load_2d(sdst, &D->tm_s[0], cg * bw, row0, bar, policy);
                                tma_load_2d(sdst + (NCW * WARP_ROWS / 2) * bw, &D->tm_s[3], cg * bw, row0, bar, policy);
                            } else {
                                tma_load_2d(sdst, &D->tm_s[sg], cg * bw, row0, bar, policy);
                            }
                        }
                        for (int bx = 0; bx < nb; ++bx) {
                            const int x = cg * kcb + bx * 128;
                            if (dual) {
                                tma_load_2d(dst + bx * CTA_BOX, &D->tm[0], x, row0, bar, policy);
                                tma_load_2d(dst + bx * CTA_BOX + CTA_BOX / 2, &D->tm[3], x, row0, bar, policy);
                            } else {
                                tma_load_2d(dst + bx * CTA_BOX, &D->tm[sg], x, row0, bar, policy);
                            }
                        }
                    } else {
                        // the consumers take consecutive K chunks of the same rows
                        uint32_t bytes = 0;
                        for (int w = 0; w < NCW; ++w) {
                            const int c = cg * NCW + w;
                            if (c < nchunks) bytes += (uint32_t)(((min(kcb, rowbytes - c * kcb) + 127) >> 7) * BOX_BYTES + (stma ? WARP_ROWS * bw : 0));
                        }
                        mbar_arrive_expect_tx(bar, bytes + (dual ? 2u : 1u) * sc_bytes);
                        send_row_scales();
                        for (int w = 0; w < NCW; ++w) {
                            const int c = cg * NCW + w;
                            if (c >= nchunks) break;
                            if (stma) {
                                const uint32_t sdst = dst + nbox * CTA_BOX;
                                if (dual) {
                                    tma_load_2d(sdst + w * (WARP_ROWS / 2) * bw, &D->tm_s[0], c * bw, row0, bar, policy);
                                    tma_load_2d(sdst + (NCW * WARP_ROWS / 2 + w * (WARP_ROWS / 2)) * bw, &D->tm_s[3], c * bw, row0, bar, policy);
                                } else {
                                    tma_load_2d(sdst + w * WARP_ROWS * bw, &D->tm_s[sg], c * bw, row0, bar, policy);
                                }
                            }
                            const int nb = (min(kcb, rowbytes - c * kcb) + 127) >> 7;
                            for (int bx = 0; bx < nb; ++bx) {
                                const int x = c * kcb + bx * 128;
                                if (dual) {
                                    tma_load_2d(dst + bx * CTA_BOX + w * (BOX_BYTES / 2), &D->tm[0], x, row0, bar, policy);
                                    tma_load_2d(dst + bx * CTA_BOX + CTA_BOX / 2 + w * (BOX_BYTES / 2), &D->tm[3], x, row0, bar, policy);
                                } else {
                                    tma_load_2d(dst + bx * CTA_BOX + w * BOX_BYTES, &D->tm[sg], x, row0, bar, policy);
                                }
                            }
                        }
                    }
                }
            }
        }
        return;
    }

    // ================= consumer warps =================
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    if (tid == 0) {
        CState S;
        S.head = 0;
        S.n = 0u;
        S.ti = 0;
        S.failed = false;
        S.ebase = ld_relaxed_u32(P.state) * (unsigned)(nops + 1);
        S.st_src = nullptr;
        S.st_epoch = 0u;
        S.st_fmt = -1;
        S.st_norm = nullptr;
        S.st_gamma = nullptr;
        S.st_xrow = 0u;
        *reinterpret_cast<CState*>(smem + PLAN_HDR_STATE) = S;
    }

    auto next_op = [&](int after) {
        int op = after + 1;
        for (; op < nops; ++op) {
            const int2 tt = s_tiles[op];
            if (first_tile(tt.x, b, G) < tt.y) break;
        }
        return op;
    };
    // the scalar half of the next descriptor is copied to shared memory while the current operator runs
    PlanOpScalars* dbuf = reinterpret_cast<PlanOpScalars*>(smem + P.off_desc);
    auto fetch_desc = [&](int op, int which) {
        if (warp == 0 && lane < 16)
            cp_async_16(smem_u32(dbuf + which) + lane * 16, reinterpret_cast<const uint8_t*>(&P.ops[op].s) + lane * 16);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int op = next_op(-1), cur = 0;
    if (op < nops) fetch_desc(op, 0);
    while (op < nops) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        consumers_sync();  // descriptor visible; everyone has left the previous operator
        const PlanOpScalars& D = dbuf[cur];
        const int nxt = next_op(op);
        if (nxt < nops) fetch_desc(nxt, cur ^ 1);
        // tiles that split K take the sixteen-part path, as in the separate launch
        const int sel = D.fmt * 2 + (D.ksplit ? 1 : 0);
        switch (sel) {
            case FMT_FP16 * 2: run_op<FMT_FP16, false>(P, D, op, smem, tid, lane, warp); break;
            case FMT_FP16 * 2 + 1: run_op<FMT_FP16, true>(P, D, op, smem, tid, lane, warp); break;
            case FMT_INT8 * 2: run_op<FMT_INT8, false>(P, D, op, smem, tid, lane, warp); break;
            case FMT_INT8 * 2 + 1: run_op<FMT_INT8, true>(P, D, op, smem, tid, lane, warp); break;
            case FMT_Q4 * 2: run_op<FMT_Q4, false>(P, D, op, smem, tid, lane, warp); break;
            default: run_op<FMT_Q4, true>(P, D, op, smem, tid, lane, warp); break;
        }
        op = nxt;
        cur ^= 1;
    }

    // ---- the launch is over for this block; the last block to get here closes the epoch ----
    consumers_sync();
    if (tid == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(P.state + 1, 1u);
        if (prev == (unsigned)G - 1u) {
            *reinterpret_cast<volatile unsigned*>(P.state + 1) = 0u;
            *reinterpret_cast<volatile unsigned*>(P.state + 2) = 0u;
            *reinterpret_cast<volatile unsigned*>(P.state) = ld_relaxed_u32(P.state) + 1u;
        }
    }
}

}  // namespace

cudaError_t decode_plan_configure() {
    return cudaFuncSetAttribute(decode_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}


cudaError_t decode_plan_func(const void** func) {
    *func = reinterpret_cast<const void*>(decode_plan_kernel);
    return cudaSuccess;
}

}  // namespace nnb
