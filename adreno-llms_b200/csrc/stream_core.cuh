// Device-side core shared by the two weight-streaming kernels (gemv_stream.cu: one launch per
// operator; decode_plan.cu: one resident launch per run of recorded operators): shared-memory
// geometry of a pipeline stage, activation staging, the RMSNorm prologue, and the per-stage
// arithmetic of the three weight formats.  Both kernels call exactly this code on the same
// K partition, so an operator gives the same bits whichever of the two runs it.
//
// Arithmetic contract (the reference's M == 1 kernels: src/models/lfm2-5-350m/kernels/
// gemv_m1{,_int8,_q4}.cl, src/models/smollm2-135m-instruct/kernels/block_fused{,_int8}.cl):
// activations and outputs fp16, sums in fp32, int8 row scale applied once after the full-K sum,
// Q4 scale applied per 32-weight block, nibble value = nibble - 8.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nnb {

constexpr int NCW = 4;                      // consumer warps per block
constexpr int STREAM_THREADS = (NCW + 1) * 32;  // + one producer warp
constexpr int WARP_ROWS = 32;               // weight rows per consumer warp per tile
constexpr int BOX_BYTES = WARP_ROWS * 128;  // one warp's 128-byte column box (4 KB)
constexpr int CTA_BOX = NCW * BOX_BYTES;    // one column box of the whole block (16 KB)
constexpr int HDR_BYTES = 128;              // 64 B of zeros + alignment room

__host__ __device__ inline int fmt_row_bytes(int fmt, int K) { return fmt == FMT_FP16 ? K * 2 : fmt == FMT_INT8 ? K : K / 2; }

// Bytes of one pipeline stage: nbox column boxes of the block, then (Q4) the block scales of the
// stage's rows (row pitch sstride for per-lane copies; tensor copies land them densely).
__host__ __device__ inline int stage_nbox(int kcb) { return (kcb + 127) / 128; }
__host__ __device__ inline int stage_sstride(int kcb) { return kcb / 8 + 16; }
__host__ __device__ inline int stage_bytes_of(int fmt, int kcb) {
    return stage_nbox(kcb) * CTA_BOX + (fmt == FMT_Q4 ? ((NCW * WARP_ROWS * stage_sstride(kcb) + 1023) / 1024) * 1024 : 0);
}
// Staged activations.  fp16 / Q4: fp16 rows; int8: three 8-bit limb planes of a 24-bit fixed-point
// copy (row stride K + 16 bytes) followed by 192 bytes of per-row maximum and scale words.
__host__ __device__ inline int x_stride_of(int fmt, int K) { return fmt == FMT_INT8 ? K + 16 : K * 2 + 16; }
__host__ __device__ inline int x_bytes_of(int fmt, int M, int K) {
    return (((fmt == FMT_INT8 ? 3 * M * x_stride_of(fmt, K) + 192 : M * x_stride_of(fmt, K)) + 127) / 128) * 128;
}
// Q4: per 32-weight block and token pair one float4 (c0, c1, c0, c1) with c = -72 * (sum of the
// block's activations), the value the block's accumulator starts from
__host__ __device__ inline int ctab_bytes_of(int fmt, int M, int K) { return fmt == FMT_Q4 ? (K / 32) * ((M + 1) / 2) * 16 : 0; }
// two reduction buffers for the consumers that split K of one tile
__host__ __device__ inline int red_bytes_of(int nt) { return 2 * NCW * 32 * 2 * nt * 4 * 4; }
// K parts of a tile whose K is split over the consumers (see "K parts" below)
constexpr int KPARTS = 2 * NCW;

// int8 weights are multiplied on the integer tensor-core path, with no conversion of the
// weights at all: each activation row is turned into 24-bit fixed point
//   x_fix = rint(x * 2^p),  2^p chosen per row so that max|x| * 2^p is in [2^22, 2^23)
// (exact for every fp16 value within 2^12 of the row's largest magnitude, otherwise rounded
// at 2^-24 of that magnitude) and split into one signed and two unsigned 8-bit limbs.  The
// three integer dot products are exact; they are recombined in fp32 and scaled by 2^-p and
// the weight row's scale.  A row holding Inf or NaN is flagged and produces NaN.
// Layout: limb planes [3][M][K + 16] (natural k order), then 16 row-maximum words (which the
// caller has cleared) and 16 floats 2^-p.
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

// RMSNorm of a single row whose norm weight is already in registers (piece j of thread tid is the
// 16-byte piece tid + j * NCW * 32 of the weight): sum of squares, then xn[k] = half((x[k] *
// rsqrt(mean x^2 + eps)) * g[k]).  Rows of up to RMSNORM_REG * NCW * 32 * 8 values.  The weight does
// not depend on the activations, so a caller that waits for x loads it while it waits.
constexpr int RMSNORM_REG = 4;
__device__ __forceinline__ void rmsnorm_load_weight(const uint16_t* __restrict__ gw, int aK, int tid, uint4 (&gv4)[RMSNORM_REG]) {
    const int per_row = aK / 8;
#pragma unroll
    for (int j = 0; j < RMSNORM_REG; ++j) {
        const int p = tid + j * NCW * 32;
        gv4[j] = p < per_row ? *reinterpret_cast<const uint4*>(gw + p * 8) : make_uint4(0, 0, 0, 0);
    }
}
__device__ __forceinline__ void rmsnorm_one_row(const uint16_t* __restrict__ x, const uint4 (&gv4)[RMSNORM_REG], float n_eps, int aK, uint16_t* xn,
                                                float* red, int tid, int lane, int warp) {
    const int per_row = aK / 8;
    constexpr int NREG = RMSNORM_REG;
    uint4 xv4[NREG];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NREG; ++j) {
        const int p = tid + j * NCW * 32;
        xv4[j] = p < per_row ? *reinterpret_cast<const uint4*>(x + p * 8) : make_uint4(0, 0, 0, 0);
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
}

// RMSNorm prologue (src/models/smollm2-135m-instruct/kernels/rmsnorm.cl:27-104 fused into the
// projection that reads its output): sum of squares per row, then the normalised fp16 rows
// xn[m][k] = half((x[m][k] * rsqrt(mean_k x[m]^2 + eps)) * gw[k]) go to shared memory.  Called by
// the NCW consumer warps; `red` holds NCW * 16 floats; ends with the consumers' barrier.
__device__ __forceinline__ void rmsnorm_rows(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gw, float n_eps, int aM, int aK,
                                             uint16_t* xn, float* red, int tid, int lane, int warp) {
    const int per_row = aK / 8;
    if (aM == 1 && per_row <= RMSNORM_REG * NCW * 32) {
        // decode fast path: the row and the norm weight are read once and stay in registers
        uint4 gv4[RMSNORM_REG];
        rmsnorm_load_weight(gw, aK, tid, gv4);
        rmsnorm_one_row(x, gv4, n_eps, aK, xn, red, tid, lane, warp);
    } else {
        for (int m = 0; m < aM; ++m) {
            float ss = 0.f;
            for (int p = tid; p < per_row; p += NCW * 32) {
                const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * aK + p * 8);
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
                const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * aK + p * 8);
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
}

// Per-lane addresses of a consumer warp inside a pipeline stage and inside the staged activations.
// A operands live in swizzled boxes: 16-byte piece q of row r sits at
//   box(q / 8) + r * 128 + ((q % 8) ^ (r % 8)) * 16.
template <int NT>
struct LaneGeo {
    uint32_t rb_base0, rb_base1;  // this warp's two 16-row blocks inside a column box (bytes from the box start)
    uint32_t a_row_off, a_q_lane; // fp16 / int8 ldmatrix.x4: (rows 0-7, piece q) (rows 8-15, q) (rows 0-7, q+1) (rows 8-15, q+1)
    uint32_t aq_off;              // Q4 ldmatrix.x4: the four 8-row groups (both row blocks) of one 16-byte piece
    uint32_t xr;
    // B: matrix j = lane/8 (16-byte piece j of the 32-k step), row n = lane%8 (+8 per n tile)
    uint32_t b_base[NT], b_step[NT], b_plane[NT];  // b_plane: int8 only, bytes between limb planes
    const uint8_t* ctab_lane[NT];  // Q4: this lane's accumulator-start quads (token pair t of each n tile), one per 32-weight block
    int ctab_step;

    __device__ __forceinline__ uint32_t piece_addr(uint32_t sw, uint32_t off, uint32_t q) const {
        return sw + (q >> 3) * CTA_BOX + off + (((q & 7) ^ xr) << 4);
    }
};

// `two_weights`: the stage holds 16 rows of each of two weights per warp (gate rows in the first
// half of a column box, up rows in the second half) instead of 32 rows of one.
template <int FMT, int NT>
__device__ __forceinline__ void lane_geo_init(LaneGeo<NT>& L, bool two_weights, int warp, int lane, int aM, uint32_t xs_addr, int xstride,
                                              uint32_t zero_addr, const uint8_t* ctab) {
    L.rb_base0 = two_weights ? (uint32_t)(warp * (BOX_BYTES / 2)) : (uint32_t)(warp * BOX_BYTES);
    L.rb_base1 = two_weights ? (uint32_t)(CTA_BOX / 2 + warp * (BOX_BYTES / 2)) : (uint32_t)(warp * BOX_BYTES + BOX_BYTES / 2);
    L.a_row_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * 128);
    L.a_q_lane = (uint32_t)(lane >> 4);
    L.aq_off = ((lane >> 4) ? L.rb_base1 : L.rb_base0) + (uint32_t)((lane & 15) * 128);
    L.xr = (uint32_t)(lane & 7);
    const int t = lane & 3;
    const int npair = (aM + 1) / 2;
    L.ctab_step = npair * 16;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int n = (lane & 7) + nt * 8;
        const bool valid = n < aM;
        L.b_base[nt] = valid ? xs_addr + n * xstride + (lane >> 3) * 16 : zero_addr;
        L.b_step[nt] = valid ? 64u : 0u;
        L.b_plane[nt] = (FMT == FMT_INT8 && valid) ? (uint32_t)(aM * xstride) : 0u;
        L.ctab_lane[nt] = ctab + min(t + 4 * nt, npair - 1) * 16;
    }
}

// K parts.  A consumer keeps two independent fp32 accumulators and deals the units of a K chunk
// (fp16: 64-byte steps; Q4: 32-weight blocks) out to them in turn, unit u of the chunk to set u mod 2,
// so that consecutive MMAs do not wait for one another; at the end of a tile it adds set 1 to set 0.
// A tile whose K is split over the four consumers (few-row operators) therefore is the sum of eight
// K parts, part 2 * (chunk mod 4) + (unit mod 2): each consumer's two sets added first, then the four
// consumers' sums in consumer order.  The resident kernel (decode_plan.cu) gives every part a warp of
// its own, built from the same unit functions below (step_fp16 / step_int8 / block_q4_at), and adds
// the parts in the same order, hence the same bits.  int8 sums are exact integers until the tile's
// end, so how a consumer's steps are dealt out does not matter there.

// fp16: one step = 64 bytes of each row = 32 k = two MMAs per row block.  `s` counts steps from the
// start of the row (it addresses the activations), `s_in_chunk` from the start of the chunk.
template <int NT>
__device__ __forceinline__ void step_fp16(const LaneGeo<NT>& L, uint32_t sw, int s, int s_in_chunk, float (&ac)[2][NT][4]) {
    uint32_t b[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) ldsm_x4(L.b_base[nt] + s * L.b_step[nt], b[nt][0], b[nt][1], b[nt][2], b[nt][3]);
    uint32_t av[2][2][4];
    const uint32_t q = (uint32_t)s_in_chunk * 4 + L.a_q_lane;
#pragma unroll
    for (int rb = 0; rb < 2; ++rb) {
        const uint32_t off = (rb ? L.rb_base1 : L.rb_base0) + L.a_row_off;
        ldsm_x4(L.piece_addr(sw, off, q), av[rb][0][0], av[rb][0][1], av[rb][0][2], av[rb][0][3]);
        ldsm_x4(L.piece_addr(sw, off, q + 2), av[rb][1][0], av[rb][1][1], av[rb][1][2], av[rb][1][3]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                mma_16816(ac[rb][nt], av[rb][h][0], av[rb][h][1], av[rb][h][2], av[rb][h][3], b[nt][2 * h], b[nt][2 * h + 1]);
}
// K chunk c (kcb bytes of every row, cb of them valid) of the stage at `sw`.
template <int NT>
__device__ __forceinline__ void chunk_fp16(const LaneGeo<NT>& L, uint32_t sw, int c, int kcb, int cb, float (&acc)[2][2][NT][4]) {
    const int s0 = (c * kcb) / 64, ns = cb / 64;
    int u = 0;
    for (; u + 2 <= ns; u += 2) {
        step_fp16<NT>(L, sw, s0 + u, u, acc[0]);
        step_fp16<NT>(L, sw, s0 + u + 1, u + 1, acc[1]);
    }
    if (u < ns) step_fp16<NT>(L, sw, s0 + u, u, acc[0]);
}

// int8: one step = 64 bytes of each row = 64 k = two integer MMAs (k32) per row block and
// activation limb; the weights go from ldmatrix straight into the MMA.  `s` counts steps from the
// start of the row (it addresses the activations), `s_in_chunk` from the start of the chunk.
template <int NT>
__device__ __forceinline__ void step_int8(const LaneGeo<NT>& L, uint32_t sw, int s, int s_in_chunk, int (&iacc)[3][2][NT][4]) {
    uint32_t b[3][NT][4];
#pragma unroll
    for (int l = 0; l < 3; ++l)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            ldsm_x4(L.b_base[nt] + l * L.b_plane[nt] + s * L.b_step[nt], b[l][nt][0], b[l][nt][1], b[l][nt][2], b[l][nt][3]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t q = (uint32_t)s_in_chunk * 4 + 2 * h + L.a_q_lane;
#pragma unroll
        for (int rb = 0; rb < 2; ++rb) {
            uint32_t w0, w1, w2, w3;
            ldsm_x4(L.piece_addr(sw, (rb ? L.rb_base1 : L.rb_base0) + L.a_row_off, q), w0, w1, w2, w3);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                imma_16832<true>(iacc[0][rb][nt], w0, w1, w2, w3, b[0][nt][2 * h], b[0][nt][2 * h + 1]);
                imma_16832<false>(iacc[1][rb][nt], w0, w1, w2, w3, b[1][nt][2 * h], b[1][nt][2 * h + 1]);
                imma_16832<false>(iacc[2][rb][nt], w0, w1, w2, w3, b[2][nt][2 * h], b[2][nt][2 * h + 1]);
            }
        }
    }
}
template <int NT>
__device__ __forceinline__ void chunk_int8(const LaneGeo<NT>& L, uint32_t sw, int c, int kcb, int cb, int (&iacc)[3][2][NT][4]) {
    const int s0 = (c * kcb) / 64;
    for (int s = 0; s < cb / 64; ++s) step_int8<NT>(L, sw, s0 + s, s, iacc);
}

// int8: recombine the limb sums, (hi * 2^16 + mid * 2^8 + lo) * 2^-p, in fp32, into acc
template <int NT>
__device__ __forceinline__ void int8_recombine(const int (&iacc)[3][2][NT][4], float (&acc)[2][NT][4], const float* rowscale, int aM, int t) {
#pragma unroll
    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = nt * 8 + 2 * t + (i & 1);
                const float v = fmaf((float)iacc[0][rb][nt][i], 65536.f, fmaf((float)iacc[1][rb][nt][i], 256.f, (float)iacc[2][rb][nt][i]));
                acc[rb][nt][i] = m < aM ? v * rowscale[m] : 0.f;
            }
}

// Q4: one step = 16 bytes of each row = one 32-weight block = two MMAs per row block on the
// biased codes (64 + nibble), started from -72 * sum(x) of the block so that the result is
// sum((nibble - 8) x), then folded in with the block's scale.  `s` = block counted from the start of
// the row, w_addr = address of this lane's part of the block's 16-byte piece, s_lo2 / s_hi2 = the
// block's scales of rows g and g + 8 of the two row blocks.
template <int NT>
__device__ __forceinline__ void block_q4(const LaneGeo<NT>& L, int s, float (&ac)[2][NT][4], const float (&s_lo2)[2], const float (&s_hi2)[2],
                                         uint32_t w_addr) {
    uint32_t b[NT][4];
    float4 cq[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        ldsm_x4(L.b_base[nt] + s * L.b_step[nt], b[nt][0], b[nt][1], b[nt][2], b[nt][3]);
        cq[nt] = *reinterpret_cast<const float4*>(L.ctab_lane[nt] + (size_t)s * L.ctab_step);
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
}
// One block on its own: block `u` of chunk c (the resident kernel's warps take every fourth block).
// `sc_rb[rb]` = the stage's scale row of this lane's row g of row block rb (rows g + 8 are 8 * sstr
// bytes further).
template <int NT>
__device__ __forceinline__ void block_q4_at(const LaneGeo<NT>& L, uint32_t sw, int c, int kcb, int u, float (&ac)[2][NT][4],
                                            const uint8_t* const (&sc_rb)[2], int sstr) {
    float lo2[2], hi2[2];
#pragma unroll
    for (int rb = 0; rb < 2; ++rb) {
        lo2[rb] = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(sc_rb[rb] + u * 2)));
        hi2[rb] = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(sc_rb[rb] + 8 * sstr + u * 2)));
    }
    block_q4<NT>(L, (c * kcb) / 16 + u, ac, lo2, hi2, L.piece_addr(sw, L.aq_off, (uint32_t)u));
}
template <int NT>
__device__ __forceinline__ void chunk_q4(const LaneGeo<NT>& L, uint32_t sw, int c, int kcb, int cb, float (&acc)[2][2][NT][4],
                                         const uint8_t* const (&sc_rb)[2], int sstr) {
    const int g0 = (c * kcb) / 16;
    uint32_t w_xor[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) w_xor[u] = (((uint32_t)u ^ (L.xr & 3u)) << 4);
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
        const uint32_t w_grp = sw + L.aq_off + (q0 >> 3) * CTA_BOX + (((q0 & 4u) ^ (L.xr & 4u)) << 4);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float lo2[2], hi2[2];
#pragma unroll
            for (int rb = 0; rb < 2; ++rb) {
                const uint32_t wl = u < 2 ? sq[rb][0].x : sq[rb][0].y, wh = u < 2 ? sq[rb][1].x : sq[rb][1].y;
                lo2[rb] = __half2float(__ushort_as_half((uint16_t)(u & 1 ? wl >> 16 : wl & 0xFFFFu)));
                hi2[rb] = __half2float(__ushort_as_half((uint16_t)(u & 1 ? wh >> 16 : wh & 0xFFFFu)));
            }
            block_q4<NT>(L, s + u, acc[u & 1], lo2, hi2, w_grp + w_xor[u]);
        }
    }
    for (; s < s1; ++s) {
        const int u = s - g0;
        if (u & 1) block_q4_at<NT>(L, sw, c, kcb, u, acc[1], sc_rb, sstr);
        else block_q4_at<NT>(L, sw, c, kcb, u, acc[0], sc_rb, sstr);
    }
}

// Single-token finish of one output row: weight-row scale (int8), then the epilogue.
// `prev` = the fp16 bits the in-place epilogues update (residual value, or the gate).
template <int FMT>
__device__ __forceinline__ uint16_t finish_row(float v, uint16_t scale_bits, int epi, uint16_t prev) {
    // explicit roundings (no fused multiply-add across the two steps): every kernel that finishes a row
    // (single-token, batched, resident) must give the same bits
    if (FMT == FMT_INT8) v = __fmul_rn(v, __half2float(__ushort_as_half(scale_bits)));
    if (epi == EPI_RESIDUAL) {
        v = __fadd_rn(__half2float(__ushort_as_half(prev)), v);
    } else if (epi == EPI_SILU_GATE) {
        const float gt = __half2float(__ushort_as_half(prev));
        v = gt * (1.0f / (1.0f + expf(-gt))) * v;
    }
    return __half_as_ushort(__float2half_rn(v));
}
// ... and of one SwiGLU row from its gate and up sums
template <int FMT>
__device__ __forceinline__ uint16_t finish_swiglu(float gv, float uv, uint16_t gscale_bits, uint16_t uscale_bits) {
    if (FMT == FMT_INT8) {
        gv *= __half2float(__ushort_as_half(gscale_bits));
        uv *= __half2float(__ushort_as_half(uscale_bits));
    }
    const float r = (gv / (1.0f + expf(-gv))) * uv;
    return __half_as_ushort(__float2half_rn(r));
}

}  // namespace nnb
