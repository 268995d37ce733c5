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
#include "ptx.cuh"

namespace nnb {

namespace {

constexpr int NCW = 4;                      // consumer warps per block
constexpr int THREADS = (NCW + 1) * 32;     // + one producer warp
constexpr int WARP_ROWS = 32;               // weight rows per consumer warp per tile
constexpr int BOX_BYTES = WARP_ROWS * 128;  // one warp's 128-byte column box (4 KB)
constexpr int CTA_BOX = NCW * BOX_BYTES;    // one column box of the whole block (16 KB)
constexpr int HDR_BYTES = 128;              // 64 B of zeros + alignment room

__host__ __device__ inline int fmt_row_bytes(int fmt, int K) { return fmt == FMT_FP16 ? K * 2 : fmt == FMT_INT8 ? K : K / 2; }

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
    g.nbox = (kcb + 127) / 128;
    g.sstride = kcb / 8 + 16;
    g.stage_bytes = g.nbox * CTA_BOX + (fmt == FMT_Q4 ? ((NCW * WARP_ROWS * g.sstride + 1023) / 1024) * 1024 : 0);
    // fp16 / Q4: activations as fp16 rows; int8: three 8-bit limb planes of a 24-bit
    // fixed-point copy (row stride K + 16 bytes) followed by 64 bytes of per-row scale words
    g.xstride = fmt == FMT_INT8 ? K + 16 : K * 2 + 16;
    g.off_bar = 64;  // full[stages], empty[stages]
    g.off_x = HDR_BYTES + ((stages * 16 + 127) / 128) * 128;
    // Q4: per 32-weight block and token pair one float4 (c0, c1, c0, c1) with c = -72 * (sum of
    // the block's activations), the value the block's accumulator starts from
    g.off_ctab = g.off_x + (((fmt == FMT_INT8 ? 3 * M * g.xstride + 192 : M * g.xstride) + 127) / 128) * 128;
    // fused RMSNorm: the normalised fp16 activations [M][K], from which the staging then reads
    g.off_norm = g.off_ctab + (fmt == FMT_Q4 ? (K / 32) * ((M + 1) / 2) * 16 : 0);
    g.off_red = g.off_norm + (norm ? ((M * K * 2 + 127) / 128) * 128 : 0);
    g.off_ring = ((g.off_red + 2 * NCW * 32 * 2 * nt * 4 * 4 + 1023) / 1024) * 1024;  // two reduction buffers
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
#ifdef NNB_TRACE
    unsigned long long* trace;  // debug build only: per-warp phase cycle counts
    int trace_slot;
#endif
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
#ifdef NNB_TRACE
    unsigned long long* trace;
    int trace_slot;
#endif
};
__device__ __forceinline__ const CUtensorMap* scale_map(const KMaps&, int) { return nullptr; }
__device__ __forceinline__ const CUtensorMap* scale_map(const KMapsQ4& km, int i) { return &km.tm_s[i]; }
template <int FMT> struct KArgsFor { typedef KArgs type; };
template <> struct KArgsFor<FMT_Q4> { typedef KArgsQ4 type; };

// int8 weights are multiplied on the integer tensor-core path, with no conversion of the
// weights at all: each activation row is turned into 24-bit fixed point
//   x_fix = rint(x * 2^p),  2^p chosen per row so that max|x| * 2^p is in [2^22, 2^23)
// (exact for every fp16 value within 2^12 of the row's largest magnitude, otherwise rounded
// at 2^-24 of that magnitude) and split into one signed and two unsigned 8-bit limbs.  The
// three integer dot products are exact; they are recombined in fp32 and scaled by 2^-p and
// the weight row's scale.  A row holding Inf or NaN is flagged and produces NaN.
// Layout: limb planes [3][M][K + 16] (natural k order), then float 2^-p per row.
__device__ __forceinline__ void stage_x_int8(const uint16_t* __restrict__ x, int M, int K, uint8_t* xs, int xstride, int tid,
                                             int nthreads) {
    unsigned int* rowmax = reinterpret_cast<unsigned int*>(xs + 3 * M * xstride);  // [16] max |x| bits, then [16] floats
    float* rowscale = reinterpret_cast<float*>(rowmax + 16);
    const int per_row = K / 8;  // 16-byte pieces
    auto quantise_piece = [&](const uint4& v, bool bad, float up, uint8_t* l0, uint8_t* l1, uint8_t* l2, int p) {
        const unsigned int w[4] = {v.x, v.y, v.z, v.w};
        uint32_t hi[2] = {0, 0}, mid[2] = {0, 0}, lo[2] = {0, 0};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint16_t hb = (uint16_t)(i & 1 ? w[i >> 1] >> 16 : w[i >> 1] & 0xFFFFu);
            const int f = bad ? 0 : __float2int_rn(__half2float(__ushort_as_half(hb)) * up);
            hi[i >> 2] |= (uint32_t)((f >> 16) & 0xFF) << (8 * (i & 3));
            mid[i >> 2] |= (uint32_t)((f >> 8) & 0xFF) << (8 * (i & 3));
            lo[i >> 2] |= (uint32_t)(f & 0xFF) << (8 * (i & 3));
        }
        *reinterpret_cast<uint2*>(l0 + p * 8) = make_uint2(hi[0], hi[1]);
        *reinterpret_cast<uint2*>(l1 + p * 8) = make_uint2(mid[0], mid[1]);
        *reinterpret_cast<uint2*>(l2 + p * 8) = make_uint2(lo[0], lo[1]);
    };
    auto piece_max = [](const uint4& v) {
        const unsigned int w[4] = {v.x, v.y, v.z, v.w};
        unsigned int mx = 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
        return mx;
    };
    auto row_params = [&](int m, bool& bad, float& up) {
        const unsigned int mx = rowmax[m];
        bad = mx >= 0x7C00u;
        // exponent of the largest magnitude: fp16 normal 2^(e-15), subnormals counted as 2^-14
        const int e = (int)(mx >> 10) > 0 ? (int)(mx >> 10) - 15 : -14;
        const int pw = (mx == 0u || bad) ? 0 : 22 - e;  // max|x| * 2^pw < 2^23
        up = __int_as_float((127 + pw) << 23);
        if (tid == 0) rowscale[m] = bad ? __int_as_float(0x7FC00000) : __int_as_float((127 - pw) << 23);
    };
    constexpr int REG_PIECES = 4;   // rows of up to 4096 values stay in registers
    if (M == 1 && per_row <= REG_PIECES * nthreads) {
        // decode fast path: the row stays in registers between the max and the split
        uint4 v[REG_PIECES];
        unsigned int mx = 0u;
#pragma unroll
        for (int j = 0; j < REG_PIECES; ++j) {
            const int p = tid + j * nthreads;
            v[j] = p < per_row ? *reinterpret_cast<const uint4*>(x + p * 8) : make_uint4(0, 0, 0, 0);
            mx = max(mx, piece_max(v[j]));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if ((tid & 31) == 0 && mx) atomicMax(&rowmax[0], mx);
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        bool bad;
        float up;
        row_params(0, bad, up);
#pragma unroll
        for (int j = 0; j < REG_PIECES; ++j) {
            const int p = tid + j * nthreads;
            if (p < per_row) quantise_piece(v[j], bad, up, xs, xs + xstride, xs + 2 * xstride, p);
        }
        return;
    }
    for (int m = 0; m < M; ++m) {
        unsigned int mx = 0u;
        for (int p = tid; p < per_row; p += nthreads) mx = max(mx, piece_max(*reinterpret_cast<const uint4*>(x + (size_t)m * K + p * 8)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if ((tid & 31) == 0 && mx) atomicMax(&rowmax[m], mx);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    // Loads are issued in batches before the shared-memory stores that follow them: a store
    // through a byte pointer may alias anything, so a load placed after one cannot be moved
    // up by the compiler and every piece would pay its own round trip to L2.
    constexpr int BATCH = 4;
    for (int m = 0; m < M; ++m) {
        bool bad;
        float up;
        row_params(m, bad, up);
        for (int p0 = tid; p0 < per_row; p0 += BATCH * nthreads) {
            uint4 v[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                const int p = p0 + j * nthreads;
                v[j] = p < per_row ? *reinterpret_cast<const uint4*>(x + (size_t)m * K + p * 8) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                const int p = p0 + j * nthreads;
                if (p < per_row) quantise_piece(v[j], bad, up, xs + (0 * M + m) * xstride, xs + (1 * M + m) * xstride, xs + (2 * M + m) * xstride, p);
            }
        }
    }
}

// Stage the activations [M, K] fp16 into shared memory, permuted per format so
// that ldmatrix over 16-byte pieces yields B fragments in the weights' packed order:
//   fp16: identity
//   Q4  : per 32 k   -> piece j, pair t = (k 8t+j, k 8t+j+4)
template <int FMT>
__device__ __forceinline__ void stage_x(const uint16_t* __restrict__ x, int M, int K, uint8_t* xs, int xstride, float* ctab, int tid,
                                        int nthreads) {
    if (FMT == FMT_FP16) {
        const int per_row = K / 8;  // 16-byte pieces
        constexpr int BATCH = 8;    // loads first, then the stores (see stage_x_int8)
        for (int i0 = tid; i0 < M * per_row; i0 += BATCH * nthreads) {
            uint4 v[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                const int i = i0 + j * nthreads;
                v[j] = i < M * per_row ? *reinterpret_cast<const uint4*>(x + (size_t)i * 8) : make_uint4(0, 0, 0, 0);  // rows are contiguous
            }
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                const int i = i0 + j * nthreads;
                if (i < M * per_row) {
                    const int m = i / per_row, p = i - m * per_row;
                    *reinterpret_cast<uint4*>(xs + m * xstride + p * 16) = v[j];
                }
            }
        }
    } else {
        const int per_row = K / 32;
        // the four loads of the next block are issued before the stores of the current one
        // (see stage_x_int8 for why the order has to be spelled out)
        const int total = M * per_row;
        uint4 cur[4], nxt[4];
        if (tid < total) {
#pragma unroll
            for (int t = 0; t < 4; ++t) cur[t] = reinterpret_cast<const uint4*>(x + (size_t)tid * 32)[t];  // rows are contiguous
        }
        for (int i = tid; i < total; i += nthreads) {
            const int m = i / per_row, p = i - m * per_row;
            if (i + nthreads < total) {
#pragma unroll
                for (int t = 0; t < 4; ++t) nxt[t] = reinterpret_cast<const uint4*>(x + (size_t)(i + nthreads) * 32)[t];
            }
            uint32_t o[4][4];
            float bsum = 0.f;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint4 v = cur[t];  // k 8t .. 8t+7 as pairs (0,1)(2,3)(4,5)(6,7)
                const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&vv[q]));
                    bsum += f.x;
                    bsum += f.y;
                }
                o[0][t] = __byte_perm(v.x, v.z, 0x5410);  // (k0, k4)
                o[1][t] = __byte_perm(v.x, v.z, 0x7632);  // (k1, k5)
                o[2][t] = __byte_perm(v.y, v.w, 0x5410);  // (k2, k6)
                o[3][t] = __byte_perm(v.y, v.w, 0x7632);  // (k3, k7)
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(xs + m * xstride + p * 64 + j * 16) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
            // accumulator start of block p, token m: (c0, c1, c0, c1) per token pair
            float* cq = ctab + ((size_t)p * ((M + 1) / 2) + (m >> 1)) * 4 + (m & 1);
            const float nc = -Q4_BIAS * bsum;
            cq[0] = nc;
            cq[2] = nc;
            if (m == M - 1 && !(m & 1)) {  // odd token count: the pair's second column is unused
                cq[1] = 0.f;
                cq[3] = 0.f;
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) cur[t] = nxt[t];
        }
    }
}

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
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full0 + s * 8, (FMT == FMT_Q4 && !ka.scale_tma) ? 1u + NCW * 32u : 1u);
            mbar_init(empty0 + s * 8, (uint32_t)NCW);
        }
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
    // This warp's two 16-row blocks inside a column box (bytes from the box start).
    const uint32_t rb_base0 = DUAL ? (uint32_t)(warp * (BOX_BYTES / 2)) : (uint32_t)(warp * BOX_BYTES);
    const uint32_t rb_base1 = DUAL ? (uint32_t)(CTA_BOX / 2 + warp * (BOX_BYTES / 2)) : (uint32_t)(warp * BOX_BYTES + BOX_BYTES / 2);
    // A operands live in swizzled boxes: 16-byte piece q of row r sits at
    //   box(q / 8) + r * 128 + ((q % 8) ^ (r % 8)) * 16.
    // fp16 / int8 ldmatrix.x4: matrices = (rows 0-7, piece q) (rows 8-15, q) (rows 0-7, q+1) (rows 8-15, q+1)
    const uint32_t a_row_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * 128);
    const uint32_t a_q_lane = (uint32_t)(lane >> 4);
    // Q4 ldmatrix.x4: matrices = the four 8-row groups (both row blocks) of one 16-byte piece
    const uint32_t aq_off = ((lane >> 4) ? rb_base1 : rb_base0) + (uint32_t)((lane & 15) * 128);
    const uint32_t xr = (uint32_t)(lane & 7);
    auto piece_addr = [&](uint32_t sw, uint32_t off, uint32_t q) { return sw + (q >> 3) * CTA_BOX + off + (((q & 7) ^ xr) << 4); };
    // B: matrix j = lane/8 (16-byte piece j of the 32-k step), row n = lane%8 (+8 per n tile)
    uint32_t b_base[NT], b_step[NT], b_plane[NT];  // b_plane: int8 only, bytes between limb planes
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int n = (lane & 7) + nt * 8;
        const bool valid = n < aM;
        b_base[nt] = valid ? smem_u32(xs) + n * geo.xstride + (lane >> 3) * 16 : zero_addr;
        b_step[nt] = valid ? 64u : 0u;
        b_plane[nt] = (FMT == FMT_INT8 && valid) ? (uint32_t)(aM * geo.xstride) : 0u;
    }
    // Q4: this lane's accumulator-start quads (token pair t of each n tile), one per 32-weight block
    const int npair = (aM + 1) / 2;
    const int ctab_step = npair * 16;
    const uint8_t* ctab_lane[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) ctab_lane[nt] = smem + geo.off_ctab + min(t + 4 * nt, npair - 1) * 16;
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

#ifdef NNB_TRACE
    const long long tl_entry = clock64();
#endif
    pdl_launch_dependents();
    pdl_wait_prior_grid();
#ifdef NNB_TRACE
    const long long tl_wait = clock64();
#endif
    if (n_items > 0 && writer) prefetch_residual(tile_first);
    const uint16_t* x_src = a.x;
    if (a_norm) {
        // RMSNorm prologue (src/models/smollm2-135m-instruct/kernels/rmsnorm.cl:27-104 fused into the
        // projection that reads its output): sum of squares per row, then the normalised fp16 row
        // goes to shared memory and the staging below reads it from there.
        uint16_t* xn = reinterpret_cast<uint16_t*>(smem + geo.off_norm);
        const uint16_t* gw = a.norm_w;
        const float n_eps = a.norm_eps;
        const int per_row = aK / 8;
        constexpr int NREG = 4;
        if (aM == 1 && per_row <= NREG * NCW * 32) {
            // decode fast path: the row and the norm weight are read once and stay in registers
            uint4 xv4[NREG], gv4[NREG];
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < NREG; ++j) {
                const int p = tid + j * NCW * 32;
                xv4[j] = p < per_row ? *reinterpret_cast<const uint4*>(a.x + p * 8) : make_uint4(0, 0, 0, 0);
                gv4[j] = p < per_row ? *reinterpret_cast<const uint4*>(gw + p * 8) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < NREG; ++j) {
                const uint32_t wv[4] = {xv4[j].x, xv4[j].y, xv4[j].z, xv4[j].w};
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
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
            float tot = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < NCW; ++w2) tot += red[w2 * 16];
            const float inv = 1.0f / sqrtf(tot / (float)aK + n_eps);
#pragma unroll
            for (int j = 0; j < NREG; ++j) {
                const int p = tid + j * NCW * 32;
                if (p >= per_row) continue;
                const uint32_t xv[4] = {xv4[j].x, xv4[j].y, xv4[j].z, xv4[j].w}, gv[4] = {gv4[j].x, gv4[j].y, gv4[j].z, gv4[j].w};
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
        } else {
        for (int m = 0; m < aM; ++m) {
            float ss = 0.f;
            for (int p = tid; p < per_row; p += NCW * 32) {
                const uint4 v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * aK + p * 8);
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
            if (lane == 0) red[warp * 16 + m] = ss;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        for (int m = 0; m < aM; ++m) {
            float tot = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < NCW; ++w2) tot += red[w2 * 16 + m];
            const float inv = 1.0f / sqrtf(tot / (float)aK + n_eps);
            for (int p = tid; p < per_row; p += NCW * 32) {
                const uint4 v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * aK + p * 8);
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
                *reinterpret_cast<uint4*>(xn + (size_t)m * aK + p * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
        }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        x_src = xn;
    }
    if (FMT == FMT_INT8) stage_x_int8(x_src, aM, aK, xs, geo.xstride, tid, NCW * 32);
    else stage_x<FMT>(x_src, aM, aK, xs, geo.xstride, reinterpret_cast<float*>(smem + geo.off_ctab), tid, NCW * 32);
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
#ifdef NNB_TRACE
    const long long tl_x = clock64();
    long long tl_full = 0, tl_comp = 0, tl_red = 0, tl_epi = 0, tl_e0 = 0, tl_e1 = 0, tl_q[4] = {0, 0, 0, 0};
#endif

#ifdef NNB_TRACE
    long long cyc_wait = 0, cyc_comp = 0, cyc_iss = 0, cyc_rel = 0, cyc_epi = 0, cyc_t0 = clock64(), cyc_a, cyc_b;
#define CYC_BEGIN() cyc_a = clock64()
#define CYC_END(acc_) do { cyc_b = clock64(); acc_ += cyc_b - cyc_a; cyc_a = cyc_b; } while (0)
#else
#define CYC_BEGIN() do { } while (0)
#define CYC_END(acc_) do { } while (0)
#endif

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
        CYC_BEGIN();
        if (FMT == FMT_Q4 && !ka.scale_tma) {
            __syncwarp();  // every lane is done with the scale rows that are about to be refilled
            if (it + stages - 1 < n_items) issue_scales(it + stages - 1);
        }
        CYC_END(cyc_iss);
        // A wait that runs out records an error and skips the arithmetic from then on;
        // the warp still walks its items so that the block's barriers stay matched.
        if (!failed && !mbar_wait_bounded(full0 + stage * 8, phase)) {
            failed = true;
            if (lane == 0) *reinterpret_cast<volatile int*>(a_status) = 1;
        }
        CYC_END(cyc_wait);
#ifdef NNB_TRACE
        if (it == 0) tl_full = clock64();
#endif
        const uint32_t sw = ring + stage * geo.stage_bytes;
        const int cb = (failed || !active) ? 0 : min(kcb, rowbytes - c * kcb);

        if (FMT == FMT_FP16) {
            // one step = 64 bytes of each row = 32 k = two MMAs per row block
            auto step = [&](int s, float (&ac)[2][NT][4]) {
                uint32_t b[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) ldsm_x4(b_base[nt] + s * b_step[nt], b[nt][0], b[nt][1], b[nt][2], b[nt][3]);
                uint32_t av[2][2][4];
                const uint32_t q = (uint32_t)(s - (c * kcb) / 64) * 4 + a_q_lane;
#pragma unroll
                for (int rb = 0; rb < 2; ++rb) {
                    const uint32_t off = (rb ? rb_base1 : rb_base0) + a_row_off;
                    ldsm_x4(piece_addr(sw, off, q), av[rb][0][0], av[rb][0][1], av[rb][0][2], av[rb][0][3]);
                    ldsm_x4(piece_addr(sw, off, q + 2), av[rb][1][0], av[rb][1][1], av[rb][1][2], av[rb][1][3]);
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
            // one step = 64 bytes of each row = 64 k = two integer MMAs (k32) per row block and
            // activation limb; the weights go from ldmatrix straight into the MMA
            const int s0 = (c * kcb) / 64;
            for (int s = 0; s < cb / 64; ++s) {
                uint32_t b[3][NT][4];
#pragma unroll
                for (int l = 0; l < 3; ++l)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                        ldsm_x4(b_base[nt] + l * b_plane[nt] + (s0 + s) * b_step[nt], b[l][nt][0], b[l][nt][1], b[l][nt][2], b[l][nt][3]);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t q = (uint32_t)s * 4 + 2 * h + a_q_lane;
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb) {
                        uint32_t w0, w1, w2, w3;
                        ldsm_x4(piece_addr(sw, (rb ? rb_base1 : rb_base0) + a_row_off, q), w0, w1, w2, w3);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            imma_16832<true>(iacc[0][rb][nt], w0, w1, w2, w3, b[0][nt][2 * h], b[0][nt][2 * h + 1]);
                            imma_16832<false>(iacc[FMT == FMT_INT8 ? 1 : 0][rb][nt], w0, w1, w2, w3, b[1][nt][2 * h], b[1][nt][2 * h + 1]);
                            imma_16832<false>(iacc[FMT == FMT_INT8 ? 2 : 0][rb][nt], w0, w1, w2, w3, b[2][nt][2 * h], b[2][nt][2 * h + 1]);
                        }
                    }
                }
            }
        } else {
            // one step = 16 bytes of each row = one 32-weight block = two MMAs per row block on
            // the biased codes (64 + nibble), started from -72 * sum(x) of the block so that the
            // result is sum((nibble - 8) x), then folded in with the block's scale
            // scale rows of this warp's two row blocks inside the stage's scale region: the
            // cp.async path keeps each warp's 32 rows together; tensor copies land whole boxes,
            // which for two weights means all gate rows first, then all up rows
            const int sstr = ka.scale_tma ? kcb / 8 : geo.sstride;
            const int srow0 = (ka.scale_tma && DUAL) ? warp * (WARP_ROWS / 2) : warp * WARP_ROWS;
            const int srow1 = (ka.scale_tma && DUAL) ? NCW * WARP_ROWS / 2 + warp * (WARP_ROWS / 2) : warp * WARP_ROWS + 16;
            const uint8_t* scb = smem + (sw - s_base) + geo.nbox * CTA_BOX;
            const uint8_t* sc_rb[2] = {scb + (srow0 + g) * sstr, scb + (srow1 + g) * sstr};
            const int g0 = (c * kcb) / 16;
            uint32_t w_xor[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w_xor[u] = (((uint32_t)u ^ (xr & 3u)) << 4);
            auto step = [&](int s, float (&ac)[2][NT][4], const float (&s_lo2)[2], const float (&s_hi2)[2], uint32_t w_addr) {
                uint32_t b[NT][4];
                float4 cq[NT];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    ldsm_x4(b_base[nt] + s * b_step[nt], b[nt][0], b[nt][1], b[nt][2], b[nt][3]);
                    cq[nt] = *reinterpret_cast<const float4*>(ctab_lane[nt] + (size_t)s * ctab_step);
                }
                uint32_t w[4];
                ldsm_x4(w_addr, w[0], w[1], w[2], w[3]);
#pragma unroll
                for (int rb = 0; rb < 2; ++rb) {
                    uint32_t p04, p15, p26, p37, q04, q15, q26, q37;
                    q4x8_to_half2x4_biased(w[rb * 2], p04, p15, p26, p37);
                    q4x8_to_half2x4_biased(w[rb * 2 + 1], q04, q15, q26, q37);
                    const float s_lo = s_lo2[rb], s_hi = s_hi2[rb];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        float d[4];
                        mma_16816_c(d, p04, q04, p15, q15, b[nt][0], b[nt][1], cq[nt]);  // starts at -72 * sum(x)
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
                // the scales of four consecutive blocks of a row are 8 contiguous, aligned bytes
                uint2 sq[2][2];
#pragma unroll
                for (int rb = 0; rb < 2; ++rb) {
                    sq[rb][0] = *reinterpret_cast<const uint2*>(sc_rb[rb] + (s - g0) * 2);
                    sq[rb][1] = *reinterpret_cast<const uint2*>(sc_rb[rb] + 8 * sstr + (s - g0) * 2);
                }
                // four consecutive 16-byte pieces of a 128-byte swizzled row: the group's part of the
                // address once, the lane's xor pattern for piece u from a table
                const uint32_t q0 = (uint32_t)(s - g0);
                const uint32_t w_grp = sw + aq_off + (q0 >> 3) * CTA_BOX + (((q0 & 4u) ^ (xr & 4u)) << 4);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float lo2[2], hi2[2];
#pragma unroll
                    for (int rb = 0; rb < 2; ++rb) {
                        const uint32_t wl = u < 2 ? sq[rb][0].x : sq[rb][0].y, wh = u < 2 ? sq[rb][1].x : sq[rb][1].y;
                        lo2[rb] = __half2float(__ushort_as_half((uint16_t)(u & 1 ? wl >> 16 : wl & 0xFFFFu)));
                        hi2[rb] = __half2float(__ushort_as_half((uint16_t)(u & 1 ? wh >> 16 : wh & 0xFFFFu)));
                    }
                    step(s + u, acc[u & 1], lo2, hi2, w_grp + w_xor[u]);
                }
            }
            for (; s < s1; ++s) {
                float lo2[2], hi2[2];
#pragma unroll
                for (int rb = 0; rb < 2; ++rb) {
                    lo2[rb] = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(sc_rb[rb] + (s - g0) * 2)));
                    hi2[rb] = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(sc_rb[rb] + 8 * sstr + (s - g0) * 2)));
                }
                const uint32_t wa = piece_addr(sw, aq_off, (uint32_t)(s - g0));
                if (s & 1) step(s, acc[1], lo2, hi2, wa);
                else step(s, acc[0], lo2, hi2, wa);
            }
        }
        CYC_END(cyc_comp);
#ifdef NNB_TRACE
        if (it == 0) tl_comp = clock64();
#endif

        // hand the stage back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + stage * 8);
        CYC_END(cyc_rel);
        if (++stage == stages) { stage = 0; phase ^= 1u; }
        const bool has_tail = (cg == groups - 1);              // this item ends its tile
        const bool seg_end = has_tail || it == n_items - 1;    // ... or this block's share of it
        if (++cg == groups) { cg = 0; tile_s += tile_step; }
        if (!seg_end) continue;
        ++ti;

        if (FMT == FMT_INT8) {
            // recombine the limb sums: (hi * 2^16 + mid * 2^8 + lo) * 2^-p, in fp32
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int m = nt * 8 + 2 * t + (i & 1);
                        const float v = fmaf((float)iacc[0][rb][nt][i], 65536.f,
                                             fmaf((float)iacc[FMT == FMT_INT8 ? 1 : 0][rb][nt][i], 256.f, (float)iacc[FMT == FMT_INT8 ? 2 : 0][rb][nt][i]));
                        acc[0][rb][nt][i] = m < aM ? v * rowscale[m] : 0.f;
                    }
        }
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
#ifdef NNB_TRACE
        if (ti == 1) tl_red = clock64();
#endif
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
#ifdef NNB_TRACE
            if (ti == 1) tl_e0 = clock64();
#endif
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
#ifdef NNB_TRACE
            if (ti == 1 && row0 >= 0) tl_e1 = clock64();
#endif
            if (lane_rows) {
                // the token's 32 results sit in lanes 0, 4, .. 28 (rows g, g + 8 of each row block):
                // bring row L to lane L, finish it there and store the 32 rows with one instruction
                const int src = (lane & 7) * 4, sel = lane >> 3;
                const float v00 = __shfl_sync(0xffffffffu, acc[0][0][0][0], src), v01 = __shfl_sync(0xffffffffu, acc[0][0][0][2], src);
                const float v10 = __shfl_sync(0xffffffffu, acc[0][1][0][0], src), v11 = __shfl_sync(0xffffffffu, acc[0][1][0][2], src);
                float v = sel == 0 ? v00 : sel == 1 ? v01 : sel == 2 ? v10 : v11;
                const int n = row0 + lane;
                if (n < seg_n) {
                    if (FMT == FMT_INT8) v *= __half2float(__ushort_as_half(sc1));
                    if (epi == EPI_RESIDUAL) {
                        v = __half2float(__ushort_as_half(res1)) + v;
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
                            if (FMT == FMT_INT8) v *= __half2float(__ushort_as_half(sc_reg[rb][i2]));
                            if (epi == EPI_RESIDUAL) {
                                v = __half2float(__ushort_as_half((uint16_t)res_reg[rb][i2][nt][j])) + v;
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
#ifdef NNB_TRACE
                    if (ti == 1) tl_q[rb * 2 + i2] = clock64();
#endif
                }
        }
    }
#ifdef NNB_TRACE
    tl_epi = clock64();
#endif
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
#ifdef NNB_TRACE
    if (ka.trace && lane == 0 && blockIdx.x < 32) {
        unsigned long long* o = ka.trace + ((size_t)ka.trace_slot * 32 + blockIdx.x) * 8 * 8 + warp * 8;
        if (warp == 0) {
            unsigned long long* tl = ka.trace + ((size_t)ka.trace_slot * 32 + blockIdx.x) * 8 * 8 + 5 * 8;
            tl[0] = tl_wait - tl_entry; tl[1] = tl_x - tl_wait; tl[2] = tl_full - tl_x; tl[3] = tl_comp - tl_full;
            tl[4] = clock64() - tl_comp; tl[5] = tl_entry - cyc_t0; tl[6] = tl_e0 - tl_red; tl[7] = tl_e1 - tl_e0; tl[5] = tl_epi - tl_e1; tl[0] = tl_q[0] - tl_e1; tl[1] = tl_q[1] - tl_e1; tl[2] = tl_q[2] - tl_e1; tl[3] = tl_q[3] - tl_e1;
        }
        o[0] = cyc_iss; o[6] = cyc_rel; o[1] = cyc_wait; o[2] = cyc_comp; o[3] = (clock64() - cyc_t0) - cyc_wait - cyc_comp - cyc_iss - cyc_rel; o[4] = n_items; o[5] = clock64() - cyc_t0;
    }
#endif
}

inline void fill_maps(KMaps& km, const KArgs& ka) {
    for (int i = 0; i < 4; ++i) km.tm[i] = ka.tm[i];
}
inline void fill_maps(KMapsQ4& km, const KArgsQ4& ka) {
    for (int i = 0; i < 4; ++i) { km.tm[i] = ka.tm[i]; km.tm_s[i] = ka.tm_s[i]; }
}

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
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
#ifdef NNB_TRACE
    ks.trace = ka.trace; ks.trace_slot = ka.trace_slot;
#endif
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
    const bool ext = a.streamk || a.npeer > 0 || a.sig.world > 0 || a.argmax_slot != nullptr || a.seg[0].out == nullptr;
    static const bool force_ext = env_int("NNB_FORCE_EXT", 0) != 0;  // tuning aid
    if (ext || force_ext) return launch_e<FMT, NT, DUAL, 2>(ka, p, st, pdl);
    if (a.norm_w) return launch_e<FMT, NT, DUAL, 1>(ka, p, st, pdl);
    return launch_e<FMT, NT, DUAL, 0>(ka, p, st, pdl);
}

#ifdef NNB_TRACE
unsigned long long* g_trace = nullptr;
int g_trace_slots = 0, g_trace_next = 0;
#endif

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

// 2-D byte view of a weight: [rows][rowbytes], box = 128 bytes x box_rows rows, 128-byte swizzle.
bool make_weight_map(CUtensorMap* m, const void* W, int rows, int rowbytes, int box_rows) {
    return cached_byte_map(m, W, rows, rowbytes, 128, box_rows, true);
}

// 2-D byte view of a Q4 scale tensor: [rows][rowbytes], dense box of box_bytes x box_rows.
bool make_scale_map(CUtensorMap* m, const void* S, int rows, int rowbytes, int box_bytes, int box_rows) {
    if (box_bytes % 16 || box_bytes > 256 || box_rows > 256) return false;
    return cached_byte_map(m, S, rows, rowbytes, box_bytes, box_rows, false);
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

int count_tiles(const LinArgs& a, int tile_rows) {
    if (a.epi == EPI_SWIGLU) return (a.seg[0].N + tile_rows - 1) / tile_rows;
    int n = 0;
    for (int i = 0; i < a.nseg; ++i) n += (a.seg[i].N + tile_rows - 1) / tile_rows;
    return n;
}

}  // namespace

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
    return gemm_tc_configure();
}

// Shapes the streaming kernel takes: 1 <= M <= 16, rows of at least 128 bytes whose
// length is a multiple of 64 bytes (fp16: K % 32, int8: K % 64, Q4: K % 128), and
// 16-byte aligned operands.  Everything else goes to the generic kernel.
bool stream_supported(int fmt, int M, int K, const LinArgs& a) {
    if (M < 1 || M > 16) return false;
    const int rb = fmt_row_bytes(fmt, K);
    // fp16 / int8 consume a row in 64-byte steps; a Q4 step is one 16-byte block, and its scale
    // rows are copied in 4-byte pieces (two blocks), so Q4 rows only have to be whole pairs of blocks
    if (rb < 128 || (rb % (fmt == FMT_Q4 ? 32 : 64)) != 0) return false;
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

// Geometry heuristics (environment overrides NNB_KCB / NNB_KW / NNB_STAGES / NNB_CTAS are
// for tuning runs):
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
    int kw = env_int("NNB_KW", 0);
    if (kw != 1 && kw != NCW) kw = count_tiles(a, NCW * warp_rows) < 2 * sm_count && rb_cols >= 256 ? NCW : 1;
    int kcb = env_int("NNB_KCB", 0);
    if (kcb <= 0) {
        if (kw == 1) kcb = 256;
        else {
            kcb = (((rb + NCW - 1) / NCW + 127) / 128) * 128;  // one chunk per consumer when the row is short
            if (kcb > 384) kcb = 256;
        }
    }
    kcb = kcb < 128 ? 128 : kcb > 1024 ? 1024 : (kcb / 128) * 128;
    if (kcb > rb_cols) kcb = rb_cols;
    while ((size_t)make_geo(fmt, M, K, kcb, 2, nt, norm).total > smem_limit && kcb > 128) kcb -= 128;
    if ((size_t)make_geo(fmt, M, K, kcb, 2, nt, norm).total > smem_limit) { p.ok = false; return p; }
    const int ntiles = count_tiles(a, kw == 1 ? NCW * warp_rows : warp_rows);
    const int nchunks = (rb + kcb - 1) / kcb;
    const int groups = kw == 1 ? nchunks : (nchunks + NCW - 1) / NCW;
    // Ring depth and blocks per SM (measured on B200): two blocks per SM with a three-stage
    // ring stream long operators best; a block with only a few pipeline items gets a ring as
    // deep as its item count, so that the whole operator is in flight after the first request.
    int stages = env_int("NNB_STAGES", 0), per_sm = 0;
    const int cap = env_int("NNB_CTAS", 0);
    int ps_first = env_int("NNB_PS", 0);
    if (ps_first < 1 || ps_first > 4) ps_first = 2;
    if (cap == 1) ps_first = 1;
    for (int ps = ps_first; ps >= 1 && !per_sm; --ps) {
        const size_t budget = (smem_limit + 1024) / ps - 1024;
        int st = stages >= 2 && stages <= 8 ? stages : (ps >= 2 ? 4 : 6);
        while (st > 2 && (size_t)make_geo(fmt, M, K, kcb, st, nt, norm).total > budget) --st;
        if ((size_t)make_geo(fmt, M, K, kcb, st, nt, norm).total > budget) continue;
        if (!(stages >= 2 && stages <= 8)) {
            const int resident = sm_count * ps;
            const int items = ((ntiles + resident - 1) / resident) * groups;  // pipeline items of the busiest block
            if (items <= st) st = items < 2 ? 2 : items;
            else if (st > 3) st = 3;
        }
        per_sm = ps;
        p.stages = st;
    }
    if (per_sm == 0) { p.ok = false; return p; }
    stages = p.stages;
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
        int want = env_int("NNB_SK", -1);
        // (measured: it pays for the instruction-bound Q4 kernel with long rows; the int8 and fp16
        // kernels are HBM-bound, idle SM slots cost them nothing and the fix-up only adds latency)
        if (want < 0) want = (fmt == FMT_Q4 && wbytes >= ((size_t)8 << 20) && plain_eff < 0.9 && sk_eff > plain_eff + 0.05 && per_block >= 8) ? 1 : 0;
        if (want && a.sk_scratch && a.sk_flags && resident <= SK_MAX_BLOCKS && total >= resident) {
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
    static const int evict_mb = env_int("NNB_EVICT_MB", 96);  // tuning: weights above this many MB are streamed evict-first
    ka.evict_first = wbytes > ((size_t)evict_mb << 20) ? 1 : 0;
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
    if (fmt == FMT_Q4 && a.K % 256 == 0 && env_int("NNB_SCALE_TMA", 1) != 0) {
        bool ok = true;
        for (int i = 0; i < a.nseg; ++i) ok = ok && (reinterpret_cast<uintptr_t>(a.seg[i].scale) & 15) == 0;
        if (dual) ok = ok && (reinterpret_cast<uintptr_t>(a.scale2) & 15) == 0;
        const int srow = a.K / 16, bw = p.kcb / 8;
        for (int i = 0; ok && i < a.nseg; ++i) ok = make_scale_map(&ka.tm_s[i], a.seg[i].scale, a.seg[i].N, srow, bw, tile_rows);
        if (ok && dual) ok = make_scale_map(&ka.tm_s[3], a.scale2, a.seg[0].N, srow, bw, tile_rows);
        ka.scale_tma = ok ? 1 : 0;
    }
#ifdef NNB_TRACE
    ka.trace = g_trace;
    ka.trace_slot = g_trace_slots ? (g_trace_next++ % g_trace_slots) : 0;
#endif
#define GO(F)                                                                                                  \
    if (fmt == F) {                                                                                            \
        if (dual) return nt == 2 ? launch_t<F, 2, true>(ka, p, st, pdl) : launch_t<F, 1, true>(ka, p, st, pdl); \
        return nt == 2 ? launch_t<F, 2, false>(ka, p, st, pdl) : launch_t<F, 1, false>(ka, p, st, pdl);         \
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
