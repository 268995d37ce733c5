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
//   * the arithmetic is the separate launch's, call for call (stream_core.cuh) on the same K
//     partition, so a run gives the same bits as the operators launched one by one;
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

struct CState {            // consumer-side state carried from operator to operator
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
};

__device__ __forceinline__ void record_failure(const PlanParams& P, CState& S, int code) {
    S.failed = true;
    *reinterpret_cast<volatile int*>(P.status) = code;
    atomicExch(P.state + 2, 1u);
}

// Poll `nw` published words until each carries `epoch`, and leave their fp16 pairs in dst.
// Eight words per thread are in flight at a time.
__device__ __forceinline__ void poll_words(const PlanParams& P, CState& S, const unsigned long long* ll, int nw, unsigned epoch, uint32_t* dst,
                                           int tid) {
    constexpr int BATCH = 8;
    for (int base = 0; base < nw; base += NCW * 32 * BATCH) {
        unsigned long long w[BATCH];
        unsigned pending = 0u;
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
            const int idx = base + j * NCW * 32 + tid;
            w[j] = 0ull;
            if (idx < nw) {
                w[j] = ld_relaxed_u64(ll + idx);
                if ((unsigned)(w[j] >> 32) != epoch) pending |= 1u << j;
            }
        }
        if (pending && !S.failed) {
            const long long t0 = clock64();
            unsigned spins = 0;
            while (pending) {
#pragma unroll
                for (int j = 0; j < BATCH; ++j) {
                    if (pending & (1u << j)) {
                        w[j] = ld_relaxed_u64(ll + base + j * NCW * 32 + tid);
                        if ((unsigned)(w[j] >> 32) == epoch) pending &= ~(1u << j);
                    }
                }
                if (pending && (++spins & 31u) == 0u) {
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
        for (int j = 0; j < BATCH; ++j) {
            const int idx = base + j * NCW * 32 + tid;
            if (idx < nw) dst[idx] = (uint32_t)w[j];
        }
    }
}

// The fp16 value of row n from the published copy (in-place epilogues).
__device__ __forceinline__ uint16_t poll_row(const PlanParams& P, CState& S, const unsigned long long* ll, int n, unsigned epoch) {
    const unsigned long long* p = ll + (n >> 1);
    unsigned long long w = ld_relaxed_u64(p);
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
template <int FMT, bool DUAL>
__device__ __forceinline__ void run_op(const PlanParams& P, const PlanOpScalars& D, int op, CState& S, uint8_t* smem, int tid, int lane, int warp) {
    const int g = lane >> 2, t = lane & 3;
    const int G = (int)gridDim.x;
    const uint32_t s_base = smem_u32(smem);
    const uint32_t full0 = s_base + PLAN_HDR_BARS, empty0 = full0 + PLAN_SLOTS * 8;
    const int ring_off = (int)(((s_base + (uint32_t)P.off_ring + 1023u) & ~1023u) - s_base);  // tensor copies want 1 KB alignment
    const uint32_t ring = s_base + (uint32_t)ring_off;
    const volatile unsigned* s_issued = reinterpret_cast<const volatile unsigned*>(smem + PLAN_HDR_ISSUED);
    const int aK = D.K, epi = D.epi, kcb = D.kcb, nchunks = D.nchunks, groups = D.groups, rowbytes = D.rowbytes;
    const int item_bytes = D.item_bytes, nbox = D.nbox, ntiles = D.ntiles, nseg = D.nseg;
    const bool ksplit = D.ksplit != 0, scale_tma = D.scale_tma != 0;
    const int seg1_tile0 = D.seg[1].tile0, seg2_tile0 = D.seg[2].tile0;
    const unsigned epoch = S.ebase + (unsigned)D.epoch;
    const bool publish_ok = op != P.drop_publish_op;
    constexpr int warp_rows = DUAL ? 16 : WARP_ROWS;
    const int tile_rows = ksplit ? warp_rows : NCW * warp_rows;
    const int xstride = x_stride_of(FMT, aK);
    uint8_t* xs = smem + P.off_xs;
    float* red = reinterpret_cast<float*>(smem + P.off_red);

    // ---------------- activations: fetch (poll the producer's words), normalise, stage ----------------
    const void* src_id = D.x_ll ? (const void*)D.x_ll : (const void*)D.x;
    const unsigned x_epoch = D.x_ll ? S.ebase + (unsigned)D.x_epoch : 0u;
    if (!(S.st_src == src_id && S.st_epoch == x_epoch && S.st_fmt == FMT && S.st_norm == (const void*)D.norm_w)) {
        const uint16_t* x_src = D.x;
        if (D.x_ll) {
            uint32_t* xraw = reinterpret_cast<uint32_t*>(smem + P.off_xraw);
            poll_words(P, S, D.x_ll, (aK + 1) >> 1, x_epoch, xraw, tid);
            x_src = reinterpret_cast<const uint16_t*>(xraw);
        }
        if (FMT == FMT_INT8 && tid < 16) reinterpret_cast<uint32_t*>(xs + 3 * xstride)[tid] = 0u;  // the row-maximum words
        // everyone is done with the previous staging and reduction buffers; the fetched row is complete
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        if (D.norm_w) {
            uint16_t* xn = reinterpret_cast<uint16_t*>(smem + P.off_norm);
            rmsnorm_rows(x_src, D.norm_w, D.norm_eps, 1, aK, xn, red, tid, lane, warp);
            x_src = xn;
        }
        if (FMT == FMT_INT8) stage_x_int8(x_src, 1, aK, xs, xstride, tid, NCW * 32);
        else stage_x<FMT>(x_src, 1, aK, xs, xstride, reinterpret_cast<float*>(smem + P.off_ctab), tid, NCW * 32);
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        S.st_src = src_id;
        S.st_epoch = x_epoch;
        S.st_fmt = FMT;
        S.st_norm = (const void*)D.norm_w;
    }

    LaneGeo<1> lg;
    lane_geo_init<FMT, 1>(lg, DUAL, warp, lane, 1, smem_u32(xs), xstride, s_base, smem + P.off_ctab);
    const float* rowscale = reinterpret_cast<const float*>(xs + 3 * xstride + 64);
    const int wrow_off = ksplit ? 0 : warp * warp_rows;
    const bool writer = !ksplit || warp == 0;

    auto tile_segment = [&](int tile) {
        int si = 0;
        if (nseg > 1 && tile >= seg1_tile0) si = 1;
        if (nseg > 2 && tile >= seg2_tile0) si = 2;
        return si;
    };

    float acc[2][2][1][4];
    int iacc[FMT == FMT_INT8 ? 3 : 1][2][1][4];
    unsigned long long am_best = 0ull;

    for (int tile = first_tile(D.tile_start, (int)blockIdx.x, G); tile < ntiles; tile += G) {
        // ---- operands of the tile's epilogue, fetched ahead of the arithmetic ----
        uint16_t sc1 = 0, res1 = 0;
        const PlanSeg sg = D.seg[DUAL ? 0 : tile_segment(tile)];
        const int row0 = (tile - sg.tile0) * tile_rows + wrow_off;
        if (writer) {
            if (DUAL) {
                if (FMT == FMT_INT8) {
                    const int n = min(row0 + (lane & 15), sg.N - 1);
                    sc1 = sg.scale[n];
                    res1 = D.scale2[n];  // the up weight's scale rides in the spare register
                }
            } else {
                if (FMT == FMT_INT8) sc1 = sg.scale[min(row0 + lane, sg.N - 1)];
                if (epi == EPI_RESIDUAL || epi == EPI_SILU_GATE) {
                    const int n = row0 + lane;
                    if (n < sg.N) res1 = D.res_ll ? poll_row(P, S, D.res_ll, n, S.ebase + (unsigned)D.res_epoch) : D.res[n];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[u][rb][0][i] = 0.f;
        if (FMT == FMT_INT8) {
#pragma unroll
            for (int l = 0; l < 3; ++l)
#pragma unroll
                for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) iacc[l % (FMT == FMT_INT8 ? 3 : 1)][rb][0][i] = 0;
        }

        // ---- the tile's pipeline items ----
        for (int cg = 0; cg < groups; ++cg) {
            const int c = ksplit ? cg * NCW + warp : cg;
            const bool active = c < nchunks;
            const int off = ring_place(S.head, item_bytes, P.ring_bytes);
            const unsigned slot = S.n % PLAN_SLOTS, parity = (S.n / PLAN_SLOTS) & 1u;
            ++S.n;
            // A wait that runs out records an error and skips the arithmetic from then on; the warp
            // still walks its items, and still waits for every copy the producer has issued, so that
            // the block's barriers stay matched and nothing is in flight when it returns.
            if (S.n - 1u < *s_issued && !mbar_wait_bounded(full0 + slot * 8, parity, P.wait_cycles)) {
                if (lane == 0 && !S.failed) record_failure(P, S, 1);
                S.failed = true;
            }
            const uint32_t sw = ring + (uint32_t)off;
            const int cb = (S.failed || !active) ? 0 : min(kcb, rowbytes - c * kcb);
            if constexpr (FMT == FMT_FP16) {
                chunk_fp16<1>(lg, sw, c, kcb, cb, acc);
            } else if constexpr (FMT == FMT_INT8) {
                chunk_int8<1>(lg, sw, c, kcb, cb, iacc);
            } else {
                // block scales arrive by tensor copies: whole boxes, which for two weights means all
                // gate rows first, then all up rows
                const int sstr = scale_tma ? kcb / 8 : stage_sstride(kcb);
                const int srow0 = (scale_tma && DUAL) ? warp * (WARP_ROWS / 2) : warp * WARP_ROWS;
                const int srow1 = (scale_tma && DUAL) ? NCW * WARP_ROWS / 2 + warp * (WARP_ROWS / 2) : warp * WARP_ROWS + 16;
                const uint8_t* scb = smem + ring_off + off + nbox * CTA_BOX;
                const uint8_t* const sc_rb[2] = {scb + (srow0 + g) * sstr, scb + (srow1 + g) * sstr};
                chunk_q4<1>(lg, sw, c, kcb, cb, acc, sc_rb, sstr);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + slot * 8);  // hand the item's bytes back to the producer
        }
        ++S.ti;

        // ---- tile finished: limb sums (int8), the two accumulator sets, the K parts in fixed order ----
        if constexpr (FMT == FMT_INT8) int8_recombine<1>(iacc, acc[0], rowscale, 1, t);
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[0][rb][0][i] += acc[1][rb][0][i];
        if (ksplit) {
            float* buf = red + (S.ti & 1) * (NCW * 32 * 2 * 4);
            if (warp != 0) {
                float* mine = buf + (warp * 32 + lane) * (2 * 4);
#pragma unroll
                for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) mine[rb * 4 + i] = acc[0][rb][0][i];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
            if (warp == 0) {
                for (int p = 1; p < NCW; ++p) {
                    const float* o = buf + (p * 32 + lane) * (2 * 4);
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[0][rb][0][i] += o[rb * 4 + i];
                }
            }
        }
        if (!writer) continue;

        // ---- epilogue: row L of the warp's rows is finished by lane L ----
        uint16_t hv = 0;
        bool valid;
        const int n = row0 + lane;
        if (DUAL) {
            // rows g, g + 8 of the warp's 16 gate / up rows sit in lanes 0, 4, .. 28
            const int src = (lane & 7) * 4, hi = (lane >> 3) & 1;
            const float g0 = __shfl_sync(0xffffffffu, acc[0][0][0][0], src), g1 = __shfl_sync(0xffffffffu, acc[0][0][0][2], src);
            const float u0 = __shfl_sync(0xffffffffu, acc[0][1][0][0], src), u1 = __shfl_sync(0xffffffffu, acc[0][1][0][2], src);
            valid = lane < 16 && n < sg.N;
            if (valid) hv = finish_swiglu<FMT>(hi ? g1 : g0, hi ? u1 : u0, sc1, res1);
        } else {
            // the token's 32 results sit in lanes 0, 4, .. 28 (rows g, g + 8 of each row block)
            const int src = (lane & 7) * 4, sel = lane >> 3;
            const float v00 = __shfl_sync(0xffffffffu, acc[0][0][0][0], src), v01 = __shfl_sync(0xffffffffu, acc[0][0][0][2], src);
            const float v10 = __shfl_sync(0xffffffffu, acc[0][1][0][0], src), v11 = __shfl_sync(0xffffffffu, acc[0][1][0][2], src);
            const float v = sel == 0 ? v00 : sel == 1 ? v01 : sel == 2 ? v10 : v11;
            valid = n < sg.N;
            if (valid) hv = finish_row<FMT>(v, sc1, epi, res1);
        }
        if (valid && sg.out) sg.out[n] = hv;
        if (sg.ll_out) {
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
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
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
}

__global__ void __launch_bounds__(STREAM_THREADS, 1) decode_plan_kernel(const __grid_constant__ PlanParams P) {
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
            mbar_init(empty0 + s * 8, (uint32_t)NCW);
        }
        mbar_init_fence();
    }
    for (int i = tid; i < nops; i += STREAM_THREADS) s_tiles[i] = P.op_tiles[i];  // written before the launch, never by it
    __syncthreads();

    // ================= producer warp: one elected lane feeds the TMA unit =================
    if (warp == NCW) {
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
            const bool stma = fmt == FMT_Q4 && __ldg(&D->s.scale_tma) != 0;
            const int seg1_tile0 = __ldg(&D->s.seg[1].tile0), seg2_tile0 = __ldg(&D->s.seg[2].tile0);
            const uint64_t policy = __ldg(&D->s.evict_first) ? l2_policy_evict_first() : l2_policy_evict_normal();
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
                for (int cg = 0; cg < groups; ++cg) {
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
                    if (!ksplit) {
                        // one copy per 128-byte column covers the rows of all four consumers
                        const int cb = min(kcb, rowbytes - cg * kcb);
                        const int nb = (cb + 127) >> 7;
                        mbar_arrive_expect_tx(bar, (uint32_t)(nb * CTA_BOX + (stma ? NCW * WARP_ROWS * bw : 0)));
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
                        mbar_arrive_expect_tx(bar, bytes);
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
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");  // descriptor visible; everyone has left the previous operator
        const PlanOpScalars& D = dbuf[cur];
        const int nxt = next_op(op);
        if (nxt < nops) fetch_desc(nxt, cur ^ 1);
        const int sel = D.fmt * 2 + (D.dual ? 1 : 0);
        switch (sel) {
            case FMT_FP16 * 2: run_op<FMT_FP16, false>(P, D, op, S, smem, tid, lane, warp); break;
            case FMT_FP16 * 2 + 1: run_op<FMT_FP16, true>(P, D, op, S, smem, tid, lane, warp); break;
            case FMT_INT8 * 2: run_op<FMT_INT8, false>(P, D, op, S, smem, tid, lane, warp); break;
            case FMT_INT8 * 2 + 1: run_op<FMT_INT8, true>(P, D, op, S, smem, tid, lane, warp); break;
            case FMT_Q4 * 2: run_op<FMT_Q4, false>(P, D, op, S, smem, tid, lane, warp); break;
            default: run_op<FMT_Q4, true>(P, D, op, S, smem, tid, lane, warp); break;
        }
        op = nxt;
        cur ^= 1;
    }

    // ---- the launch is over for this block; the last block to get here closes the epoch ----
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
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
