// Any-shape, any-alignment linear kernel: one warp per output row.
//
// Plays the role of the reference's inline gemv_rT_fp32acc
// (src/models/lfm2-5-350m/src/utils.cpp:35-73), the only path there that takes any
// K: vec4 steps strided over the work-items, scalar tail, fp32 accumulation,
// shuffle reduction.  It is the landing place for shapes the streaming kernel does
// not take (unaligned pointers, row lengths that are not a multiple of 64 bytes,
// M > 16 slices); it reads with element-sized loads only.
#include <cuda_fp16.h>

#include "kernels.h"

namespace nnb {
namespace {

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

template <int FMT>
__device__ __forceinline__ float row_dot(const uint8_t* __restrict__ wrow, const uint16_t* __restrict__ srow,
                                         const uint16_t* __restrict__ x, int K, int lane) {
    float acc = 0.f;
    if (FMT == FMT_Q4) {
        // one 8-nibble group per lane per step; the block scale folds in per group
        const int npix = K >> 3;
        for (int pix = lane; pix < npix; pix += 32) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint8_t b = wrow[pix * 4 + i];
                d += h2f(x[pix * 8 + 2 * i]) * (float)((int)(b & 0xF) - 8);
                d += h2f(x[pix * 8 + 2 * i + 1]) * (float)((int)(b >> 4) - 8);
            }
            acc += d * h2f(srow[pix >> 2]);
        }
    } else {
        const int K4 = K >> 2;
        for (int k4 = lane; k4 < K4; k4 += 32) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = 4 * k4 + i;
                const float w = FMT == FMT_FP16 ? h2f(reinterpret_cast<const uint16_t*>(wrow)[k])
                                                : (float)reinterpret_cast<const int8_t*>(wrow)[k];
                d += h2f(x[k]) * w;
            }
            acc += d;
        }
        for (int k = K4 * 4 + lane; k < K; k += 32) {
            const float w = FMT == FMT_FP16 ? h2f(reinterpret_cast<const uint16_t*>(wrow)[k])
                                            : (float)reinterpret_cast<const int8_t*>(wrow)[k];
            acc += h2f(x[k]) * w;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    return acc;
}

template <int FMT>
__global__ void linear_generic_kernel(const __grid_constant__ LinArgs a, int total_rows) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const size_t rowbytes = FMT == FMT_FP16 ? (size_t)a.K * 2 : FMT == FMT_INT8 ? (size_t)a.K : (size_t)a.K / 2;
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < total_rows; r += gridDim.x * wpb) {
        int si = 0, n = r;
        while (si + 1 < a.nseg && n >= a.seg[si].N) { n -= a.seg[si].N; ++si; }
        const LinSeg& sg = a.seg[si];
        const uint8_t* wrow = sg.W + rowbytes * n;
        const uint16_t* srow = FMT == FMT_Q4 ? sg.scale + (size_t)n * (a.K / 32) : nullptr;
        for (int m = 0; m < a.M; ++m) {
            const uint16_t* xm = a.x + (size_t)m * a.K;
            float v = row_dot<FMT>(wrow, srow, xm, a.K, lane);
            if (FMT == FMT_INT8) v *= h2f(sg.scale[n]);
            uint16_t* o = sg.out + (size_t)m * sg.ld_out + n;
            if (a.epi == EPI_SWIGLU) {
                const uint8_t* urow = a.W2 + rowbytes * n;
                const uint16_t* usrow = FMT == FMT_Q4 ? a.scale2 + (size_t)n * (a.K / 32) : nullptr;
                float u = row_dot<FMT>(urow, usrow, xm, a.K, lane);
                if (FMT == FMT_INT8) u *= h2f(a.scale2[n]);
                v = (v / (1.0f + expf(-v))) * u;
            } else if (a.epi == EPI_RESIDUAL) {
                v = h2f(*o) + v;
            } else if (a.epi == EPI_SILU_GATE) {
                const float gt = h2f(*o);
                v = gt * (1.0f / (1.0f + expf(-gt))) * v;
            }
            if (lane == 0) *o = __half_as_ushort(__float2half_rn(v));
        }
    }
}

}  // namespace

cudaError_t launch_generic(int fmt, const LinArgs& a, cudaStream_t st) {
    int rows = 0;
    for (int i = 0; i < a.nseg; ++i) rows += a.seg[i].N;
    if (rows == 0 || a.M == 0) return cudaSuccess;
    const int threads = 256, wpb = threads / 32;
    int grid = (rows + wpb - 1) / wpb;
    const int cap = current_sm_count() * 8;
    if (grid > cap) grid = cap;
    if (fmt == FMT_FP16) linear_generic_kernel<FMT_FP16><<<grid, threads, 0, st>>>(a, rows);
    else if (fmt == FMT_INT8) linear_generic_kernel<FMT_INT8><<<grid, threads, 0, st>>>(a, rows);
    else linear_generic_kernel<FMT_Q4><<<grid, threads, 0, st>>>(a, rows);
    return cudaGetLastError();
}

}  // namespace nnb
