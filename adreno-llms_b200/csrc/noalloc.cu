// nn_argmax_static: arg-max over fp16 logits for callers that must not allocate.
//
// nn_argmax keeps its 8-byte reduction slot in memory obtained with cudaMalloc when the
// context is created.  Some hosts of this library cannot do that: a sampler callback invoked
// from a real-time audio or UI thread that works under a no-allocation rule, an embedding
// application that has handed the whole device heap to its own pool allocator and forbids
// third-party cudaMalloc, or a service whose device-memory budget is frozen once start-up is
// over.  This entry point needs no context and no heap: its
// scratch lives in a file-scope __device__ array that every GPU loading the library carries
// from load until exit (256 bytes).
//
// Limits and rules
//   * n <= NN_ARGMAX_STATIC_MAX_N logits per call; larger n is refused with NN_ERR_ARG.
//   * The first call on each device looks up the device address of the scratch array
//     (cudaGetSymbolAddress); make that first call outside any stream capture.
//   * Every call on a device shares the one scratch array.  The call clears the slot it uses
//     before reducing into it, so stale contents never leak into a result, but two calls
//     that overlap on the GPU (different streams, no ordering between them) race on it.
//     Calls ordered on one stream are safe.
//   * It calls no cudaMalloc / cudaFree and no allocating library routine.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/nnopt_b200.h"
#include "internal.h"
#include "kernels.h"

namespace {

constexpr int kSlots = 32;  // 256 bytes; slot 0 is the reduction word, the rest is spare
static __device__ __align__(256) unsigned long long g_static_scratch[kSlots];

constexpr int kMaxDevices = 64;
std::atomic<unsigned long long*> g_scratch_addr[kMaxDevices];  // device address per device, filled on first use (any thread)

__device__ __forceinline__ unsigned long long key_of(float v, int idx) {
    unsigned int b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)idx);
}

__global__ void static_clear_kernel(unsigned long long* slot) { *slot = 0ull; }

__global__ void static_argmax_kernel(const uint16_t* __restrict__ v, int n, unsigned long long* slot) {
    unsigned long long best = 0ull;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float f = __half2float(__ushort_as_half(v[i]));
        if (f == f) {
            const unsigned long long k = key_of(f, i);
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

__global__ void static_finish_kernel(const unsigned long long* slot, int* out_idx) {
    const unsigned long long k = *slot;
    *out_idx = k ? (int)(0xFFFFFFFFu - (unsigned int)(k & 0xFFFFFFFFull)) : -1;
}

}  // namespace

extern "C" int nn_argmax_static(void* cuda_stream, int n, nn_buf logits_fp16, nn_buf out_index_i32) {
    if (!logits_fp16 || !out_index_i32) return NN_FAIL(NN_ERR_ARG, "nn_argmax_static: null buffer");
    if (n < 0 || n > NN_ARGMAX_STATIC_MAX_N)
        return NN_FAIL(NN_ERR_ARG, "nn_argmax_static: n=%d is outside [0, %d], the size this allocation-free entry point is built for", n,
                       NN_ARGMAX_STATIC_MAX_N);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return NN_FAIL(NN_ERR_CUDA, "nn_argmax_static: no current CUDA device (%s)", cudaGetErrorString(e));
    unsigned long long* slot = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!slot) {
        // Once per device, with that device current: the array's name is only a host-side
        // handle; the kernels need its device address.
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return NN_FAIL(NN_ERR_CUDA, "nn_argmax_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        slot = static_cast<unsigned long long*>(p);
        g_scratch_addr[dev].store(slot, std::memory_order_release);   // every thread computes the same value
    }
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    static_clear_kernel<<<1, 1, 0, st>>>(slot);
    if (n > 0) {
        int blocks = (n + 1023) / 1024;
        const int cap = nnb::current_sm_count() * 4;
        if (blocks > cap) blocks = cap;
        static_argmax_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(logits_fp16), n, slot);
    }
    static_finish_kernel<<<1, 1, 0, st>>>(slot, static_cast<int*>(out_index_i32));
    e = cudaGetLastError();
    if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "nn_argmax_static: launch failed: %s", cudaGetErrorString(e));
    return NN_OK;
}
