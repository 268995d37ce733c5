// Small helper kernels: dequantisation dump (parity check of the unpack rule),
// arg-max over fp16 logits, L2 flush for cold timing.
#include <cuda_fp16.h>
#include <float.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nnb {
namespace {

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// out[n,k] = float(code) * float(scale): the unpack contract of
// src/models/lfm2-5-350m/kernels/gemv_m1_q4.cl:31-40 (nibble - 8, low nibble = even k)
// and src/models/lfm2-5-350m/scripts/quantize_weights.py:136 (int8 * per-row scale).
template <int FMT>
__global__ void dequant_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ scale, float* __restrict__ out,
                               int N, int K) {
    const size_t total = (size_t)N * K;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / K;
        const int k = (int)(i - n * K);
        float v;
        if (FMT == FMT_FP16) {
            v = h2f(reinterpret_cast<const uint16_t*>(W)[i]);
        } else if (FMT == FMT_INT8) {
            v = (float)reinterpret_cast<const int8_t*>(W)[i] * h2f(scale[n]);
        } else {
            const uint8_t b = W[n * (size_t)(K / 2) + (k >> 1)];
            const int code = (int)((b >> (4 * (k & 1))) & 0xF) - 8;
            v = (float)code * h2f(scale[n * (size_t)(K / 32) + (k >> 5)]);
        }
        out[i] = v;
    }
}

// Order-preserving key: larger value wins, then the LOWER index.
__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
    unsigned int b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)idx);
}

__global__ void argmax_half_kernel(const uint16_t* __restrict__ v, int n, unsigned long long* slot) {
    unsigned long long best = 0ull;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float f = h2f(v[i]);
        if (f == f) {  // NaNs never win
            const unsigned long long k = argmax_key(f, i);
            best = k > best ? k : best;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    __shared__ unsigned long long sm[32];
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? sm[threadIdx.x] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (threadIdx.x == 0 && best) atomicMax(slot, best);
    }
}

__global__ void fill_u64_kernel(unsigned long long* p, unsigned long long v) { *p = v; }

__global__ void argmax_finish_kernel(const unsigned long long* slot, int* out_idx) {
    const unsigned long long k = *slot;
    *out_idx = k ? (int)(0xFFFFFFFFu - (unsigned int)(k & 0xFFFFFFFFull)) : -1;
}

// RMSNorm on fp16 storage, one block per row: out = half((x * rsqrt(mean(x^2) + eps)) * weight)
// (src/models/smollm2-135m-instruct/kernels/rmsnorm.cl:27-104; fp32 sums, a different but fixed order).
__global__ void rmsnorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, uint16_t* __restrict__ out, int cols, float eps) {
    const uint16_t* xr = x + (size_t)blockIdx.x * cols;
    uint16_t* orow = out + (size_t)blockIdx.x * cols;
    float ss = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = h2f(xr[c]);
        ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __shared__ float part[32];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += part[i];
    const float inv = 1.0f / sqrtf(tot / (float)cols + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) orow[c] = __half_as_ushort(__float2half_rn((h2f(xr[c]) * inv) * h2f(w[c])));
}

// out[r][c] = half(float(out[r][c]) + float(bias[c])) for up to three (out, bias) pairs of one launch:
// bias_add_rowmajor, src/models/qwen2-5-0-5b/kernels/bias_add.cl:18-40 (the projection's result is
// rounded to fp16 first, then the bias is added in fp32 and the sum rounded again, as there).
__global__ void bias_add_kernel(BiasArgs a) {
    const int seg = blockIdx.y;
    uint16_t* out = a.out[seg];
    const uint16_t* bias = a.bias[seg];
    const int cols = a.cols[seg];
    const long long total = (long long)a.rows * cols;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % cols);
        out[i] = __half_as_ushort(__float2half_rn(h2f(out[i]) + h2f(bias[c])));
    }
}

// Read-bandwidth probes: what the weight streams of this library can reach at best on this GPU
// (the role of gemv_stream_buf / gemv_stream_img, src/models/lfm2-5-350m/kernels/gemv_m1.cl:537-589,
// driven by run_bw_probe, src/models/lfm2-5-350m/src/main.cpp:29-139).  The two read paths of this
// hardware stand where the reference has buffer and image reads: 16-byte loads by every thread, and
// bulk copies into shared memory by the TMA unit (the path the streaming kernels use).
__global__ void __launch_bounds__(256) probe_loads_kernel(const uint4* __restrict__ src, size_t n16, float* __restrict__ sink) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    unsigned int acc = 0u;
    constexpr int U = 8;  // independent loads in flight per thread
    for (; i + (U - 1) * stride < n16; i += U * stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                         : "l"(src + i + u * stride));
#pragma unroll
        for (int u = 0; u < U; ++u) acc += v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    for (; i < n16; i += stride) {
        const uint4 v = src[i];
        acc += v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9E3779B9u) sink[threadIdx.x] = 1.f;  // keeps the loads alive; practically never taken
}

constexpr int PROBE_CHUNK = 16384;
constexpr int PROBE_STAGES = 8;

__global__ void __launch_bounds__(32) probe_tma_kernel(const uint8_t* __restrict__ src, size_t nchunks, unsigned* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t probe_smem[];
    __shared__ __align__(8) uint64_t bars[PROBE_STAGES];
    if (threadIdx.x != 0) return;
    for (int s = 0; s < PROBE_STAGES; ++s) mbar_init(smem_u32(&bars[s]), 1);
    mbar_init_fence();
    const uint64_t pol = l2_policy_evict_first();
    size_t issued = 0, waited = 0;   // per stage ring: copy number i lands in stage i % PROBE_STAGES
    bool ok = true;
    for (size_t c = blockIdx.x; c < nchunks && ok; c += gridDim.x) {
        if (issued >= PROBE_STAGES) {  // the copy that used this stage before must have landed
            ok = mbar_wait_bounded(smem_u32(&bars[waited % PROBE_STAGES]), (uint32_t)((waited / PROBE_STAGES) & 1));
            if (!ok) break;
            ++waited;
        }
        const int s = (int)(issued % PROBE_STAGES);
        mbar_arrive_expect_tx(smem_u32(&bars[s]), PROBE_CHUNK);
        bulk_g2s(smem_u32(probe_smem + (size_t)s * PROBE_CHUNK), src + c * (size_t)PROBE_CHUNK, PROBE_CHUNK, smem_u32(&bars[s]), pol);
        ++issued;
    }
    // every copy in flight lands before the block gives its shared memory back (bounded as well)
    for (; waited < issued; ++waited)
        if (!mbar_wait_bounded(smem_u32(&bars[waited % PROBE_STAGES]), (uint32_t)((waited / PROBE_STAGES) & 1))) ok = false;
    if (!ok) atomicExch(status, 1u);
}

// The element-wise halves of the two-weight forms at prefill row counts, where each projection is a tensor-core GEMM of
// its own with an fp16 result, as in the reference (its M > 1 path runs w1, w3 and then a SiLU-multiply kernel over the
// fp16 results: src/models/lfm2-5-350m/src/layers/mlp.cpp:101-129, kernels/mlp.cl:6):
//   out[i]  = half(silu(float(g[i])) * float(u[i]))          (g may be out: the in-place gate form)
__global__ void silu_mul_kernel(const uint16_t* __restrict__ g, const uint16_t* __restrict__ u, uint16_t* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float gv = h2f(g[i]), uv = h2f(u[i]);
        out[i] = __half_as_ushort(__float2half_rn((gv / (1.0f + expf(-gv))) * uv));
    }
}

__global__ void l2_flush_kernel(uint4* buf, size_t n16) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        uint4 v = buf[i];
        v.x += 1u;
        buf[i] = v;
    }
}

}  // namespace

int current_sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 132;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 132;
        cached[dev] = n;
    }
    return cached[dev];
}

cudaError_t launch_dequant(int fmt, int N, int K, const void* W, const uint16_t* scale, float* out, cudaStream_t st) {
    const size_t total = (size_t)N * K;
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    const size_t cap = (size_t)current_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    const uint8_t* w = static_cast<const uint8_t*>(W);
    if (fmt == FMT_FP16) dequant_kernel<FMT_FP16><<<(unsigned)blocks, threads, 0, st>>>(w, scale, out, N, K);
    else if (fmt == FMT_INT8) dequant_kernel<FMT_INT8><<<(unsigned)blocks, threads, 0, st>>>(w, scale, out, N, K);
    else dequant_kernel<FMT_Q4><<<(unsigned)blocks, threads, 0, st>>>(w, scale, out, N, K);
    return cudaGetLastError();
}

cudaError_t launch_fill_u64(unsigned long long* p, unsigned long long v, cudaStream_t st) {
    fill_u64_kernel<<<1, 1, 0, st>>>(p, v);
    return cudaGetLastError();
}

cudaError_t launch_argmax_finish(const unsigned long long* slot, int* out_idx, cudaStream_t st) {
    argmax_finish_kernel<<<1, 1, 0, st>>>(slot, out_idx);
    return cudaGetLastError();
}

cudaError_t launch_argmax_half(const uint16_t* v, int n, int* out_idx, unsigned long long* slot, cudaStream_t st) {
    cudaError_t e = launch_fill_u64(slot, 0ull, st);
    if (e != cudaSuccess) return e;
    if (n > 0) {
        int blocks = (n + 1023) / 1024;
        const int cap = current_sm_count() * 4;
        if (blocks > cap) blocks = cap;
        argmax_half_kernel<<<blocks, 256, 0, st>>>(v, n, slot);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    return launch_argmax_finish(slot, out_idx, st);
}

cudaError_t launch_rmsnorm(const uint16_t* x, const uint16_t* w, uint16_t* out, int rows, int cols, float eps, cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    rmsnorm_kernel<<<(unsigned)rows, 256, 0, st>>>(x, w, out, cols, eps);
    return cudaGetLastError();
}

cudaError_t launch_bias_add(const BiasArgs& a, cudaStream_t st) {
    if (a.rows <= 0 || a.nseg <= 0) return cudaSuccess;
    int maxc = 0;
    for (int i = 0; i < a.nseg; ++i) maxc = a.cols[i] > maxc ? a.cols[i] : maxc;
    long long blocks = ((long long)a.rows * maxc + 255) / 256;
    const long long cap = (long long)current_sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    bias_add_kernel<<<dim3((unsigned)blocks, (unsigned)a.nseg), 256, 0, st>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_probe_loads(const void* src, size_t bytes, float* sink, cudaStream_t st) {
    probe_loads_kernel<<<current_sm_count() * 8, 256, 0, st>>>(static_cast<const uint4*>(src), bytes / 16, sink);
    return cudaGetLastError();
}

cudaError_t launch_probe_tma(const void* src, size_t bytes, unsigned* status, cudaStream_t st) {
    static bool configured = false;
    const int smem = PROBE_CHUNK * PROBE_STAGES;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(probe_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    probe_tma_kernel<<<current_sm_count(), 32, smem, st>>>(static_cast<const uint8_t*>(src), bytes / PROBE_CHUNK, status);
    return cudaGetLastError();
}

cudaError_t launch_silu_mul(const uint16_t* g, const uint16_t* u, uint16_t* out, size_t n, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    size_t blocks = (n + 1023) / 1024;
    const size_t cap = (size_t)current_sm_count() * 8;
    if (blocks > cap) blocks = cap;
    silu_mul_kernel<<<(unsigned)blocks, 256, 0, st>>>(g, u, out, n);
    return cudaGetLastError();
}

cudaError_t launch_l2_flush(void* buf, size_t bytes, cudaStream_t st) {
    const size_t n16 = bytes / 16;
    if (!n16) return cudaSuccess;
    l2_flush_kernel<<<(unsigned)current_sm_count() * 8u, 256, 0, st>>>(static_cast<uint4*>(buf), n16);
    return cudaGetLastError();
}

}  // namespace nnb
