// Activations of a batched call (2 <= M <= 16) staged ONCE per launch.
//
// The streaming kernel keeps the whole activation batch in shared memory in a per-format staged
// form (int8: three limb planes of a per-row 24-bit fixed-point copy plus the row scales; Q4: rows
// permuted for ldmatrix plus the table of -72 * (sum of a block's activations); fp16: the rows).
// With one token every block builds that form itself out of a few KB.  With M rows the same work
// (up to 230 KB of output) repeated by every block of the launch is what bounds batched decode, so
// a small grid, one block per activation row, writes the staged image (byte for byte the shared-
// memory layout) to context scratch, and every block of the projection pulls it with one bulk copy.
// The optional RMSNorm of the rows (rmsnorm_forward, src/models/smollm2-135m-instruct/kernels/
// rmsnorm.cl:27-104) is applied here, once, instead of by every block.
//
// The reference has no batched GEMV (quantised M > 1 is a loop of M = 1 calls,
// src/models/lfm2-5-350m/src/model.cpp:243-251); the arithmetic per row is that of the single-token
// path.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "ptx.cuh"
#include "stream_core.cuh"

namespace nnb {
namespace {

constexpr int ST = NCW * 32;  // threads per block: the norm helpers synchronise exactly this many

template <int FMT>
__global__ void __launch_bounds__(ST) stage_image_kernel(const uint16_t* __restrict__ x, int M, int K, const uint16_t* __restrict__ norm_w,
                                                        float eps, uint8_t* __restrict__ img) {
    extern __shared__ __align__(16) uint8_t st_smem[];  // the normalised row, when there is a norm
    __shared__ float red[NCW * 16];
    __shared__ unsigned int wmax[NCW];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, m = blockIdx.x;
    pdl_launch_dependents();  // the projection may start fetching weights; it waits for this grid before it reads the image
    pdl_wait_prior_grid();    // the rows may come from the launch before, which may also still read the image
    const uint16_t* row = x + (size_t)m * K;
    if (norm_w) {
        uint16_t* xn = reinterpret_cast<uint16_t*>(st_smem);
        rmsnorm_rows(row, norm_w, eps, 1, K, xn, red, tid, lane, warp);
        row = xn;
    }
    const int xstride = x_stride_of(FMT, K);
    if (FMT == FMT_FP16) {
        uint8_t* dst = img + (size_t)m * xstride;
        for (int p = tid; p < K / 8; p += ST) *reinterpret_cast<uint4*>(dst + p * 16) = *reinterpret_cast<const uint4*>(row + p * 8);
    } else if (FMT == FMT_INT8) {
        // the row's largest magnitude, then 24-bit fixed point in three 8-bit limbs (see stage_x_int8)
        const int per_row = K / 8;
        unsigned int mx = 0u;
        for (int p = tid; p < per_row; p += ST) {
            const uint4 v = *reinterpret_cast<const uint4*>(row + p * 8);
            const unsigned int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) wmax[warp] = mx;
        __syncthreads();
        mx = 0u;
#pragma unroll
        for (int w2 = 0; w2 < NCW; ++w2) mx = max(mx, wmax[w2]);
        const bool bad = mx >= 0x7C00u;
        const int e = (int)(mx >> 10) > 0 ? (int)(mx >> 10) - 15 : -14;
        const int pw = (mx == 0u || bad) ? 0 : 22 - e;
        const float up = __int_as_float((127 + pw) << 23);
        unsigned int* rowmax = reinterpret_cast<unsigned int*>(img + (size_t)3 * M * xstride);
        float* rowscale = reinterpret_cast<float*>(rowmax + 16);
        if (tid == 0) {
            rowmax[m] = mx;
            rowscale[m] = bad ? __int_as_float(0x7FC00000) : __int_as_float((127 - pw) << 23);
        }
        uint8_t* l0 = img + (size_t)(0 * M + m) * xstride;
        uint8_t* l1 = img + (size_t)(1 * M + m) * xstride;
        uint8_t* l2 = img + (size_t)(2 * M + m) * xstride;
        for (int p = tid; p < per_row; p += ST) {
            const uint4 v = *reinterpret_cast<const uint4*>(row + p * 8);
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
        }
    } else {
        // Q4: per 32 k, piece j holds the pairs (k 8t+j, k 8t+j+4), t = 0..3; the block's accumulator
        // start -72 * (sum of the block's activations) goes to the table (see stage_x)
        const int per_row = K / 32;
        uint8_t* dst = img + (size_t)m * xstride;
        float* ctab = reinterpret_cast<float*>(img + x_bytes_of(FMT_Q4, M, K));
        for (int p = tid; p < per_row; p += ST) {
            uint4 cur[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) cur[t] = reinterpret_cast<const uint4*>(row + (size_t)p * 32)[t];
            uint32_t o[4][4];
            float bsum = 0.f;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint4 v = cur[t];
                const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&vv[q]));
                    bsum += f.x;
                    bsum += f.y;
                }
                o[0][t] = __byte_perm(v.x, v.z, 0x5410);
                o[1][t] = __byte_perm(v.x, v.z, 0x7632);
                o[2][t] = __byte_perm(v.y, v.w, 0x5410);
                o[3][t] = __byte_perm(v.y, v.w, 0x7632);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(dst + p * 64 + j * 16) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
            float* cq = ctab + ((size_t)p * ((M + 1) / 2) + (m >> 1)) * 4 + (m & 1);
            const float nc = -Q4_BIAS * bsum;
            cq[0] = nc;
            cq[2] = nc;
            if (m == M - 1 && !(m & 1)) {
                cq[1] = 0.f;
                cq[3] = 0.f;
            }
        }
    }
}

}  // namespace

size_t stage_image_bytes(int fmt, int M, int K) { return (size_t)x_bytes_of(fmt, M, K) + (size_t)ctab_bytes_of(fmt, M, K); }

cudaError_t launch_stage_image(int fmt, const uint16_t* x, int M, int K, const uint16_t* norm_w, float eps, uint8_t* img, cudaStream_t st,
                               bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)M);
    cfg.blockDim = dim3((unsigned)ST);
    cfg.dynamicSmemBytes = norm_w ? (size_t)K * 2 : 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (fmt == FMT_FP16) return cudaLaunchKernelEx(&cfg, stage_image_kernel<FMT_FP16>, x, M, K, norm_w, eps, img);
    if (fmt == FMT_INT8) return cudaLaunchKernelEx(&cfg, stage_image_kernel<FMT_INT8>, x, M, K, norm_w, eps, img);
    if (fmt == FMT_Q4) return cudaLaunchKernelEx(&cfg, stage_image_kernel<FMT_Q4>, x, M, K, norm_w, eps, img);
    return cudaErrorInvalidValue;
}

}  // namespace nnb
