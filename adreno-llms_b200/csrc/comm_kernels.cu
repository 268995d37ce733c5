// Cross-rank completion flags for the row-sharded gather, in peer-mapped device memory.
//
// After a rank's projection kernel has stored its [M, N/G] block into every rank's gather
// buffer (plain peer stores over NVLink), comm_signal_kernel publishes a new epoch number in
// word `rank` of every rank's flag array, and comm_wait_kernel on each rank holds the stream
// until all G words of its own array have reached its epoch.  Both epochs live in device
// memory and advance by one per launch, so the pair can be recorded into a plan and replayed.
//
// The wait is bounded by wall time (%globaltimer): when it runs out the kernel writes a
// status word that nn_sync reports as NN_ERR_TIMEOUT, and returns; the context stays usable.
//
// comm_pick_kernel finishes a row-sharded greedy pick.  Each rank's projection kernel leaves one
// 64-bit word with every rank: pick number (16 bits) | ordered fp16 value (16) | ~row (32).  The
// word is its own flag (an aligned 8-byte store arrives whole), so the exchange needs no fence:
// the kernel spins until all G words of this pick's table carry the pick's number and takes the
// largest.  The logits never leave the rank that computed them.
// The reference is single-device and has no counterpart of this file.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace nnb {
namespace {

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void comm_signal_kernel(PeerFlags pf, unsigned* epoch_sent) {
    __shared__ unsigned e;
    if (threadIdx.x == 0) {
        e = *epoch_sent + 1u;
        *epoch_sent = e;
    }
    __syncthreads();
    // the stores of the kernels before this one in the stream are ordered before the flag
    if ((int)threadIdx.x < pf.world) {
        unsigned* dst = pf.flags[threadIdx.x] + pf.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(e) : "memory");
    }
}

__global__ void comm_wait_kernel(const unsigned* my_flags, int world, unsigned* epoch_waited, unsigned timeout_ms, int* status) {
    __shared__ unsigned e;
    if (threadIdx.x == 0) {
        e = *epoch_waited + 1u;
        *epoch_waited = e;
    }
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const unsigned long long t0 = global_ns();
        const unsigned long long limit = (unsigned long long)timeout_ms * 1000000ull;
        const unsigned* src = my_flags + threadIdx.x;
        for (;;) {
            unsigned v;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
            if ((int)(v - e) >= 0) break;
            if (global_ns() - t0 > limit) {
                *reinterpret_cast<volatile int*>(status) = 7;
                break;
            }
            __nanosleep(32);
        }
    }
    // one acquire for all the flags read above: what the signalling ranks stored before their
    // flags is visible to the kernels that follow in this stream
    asm volatile("fence.acq_rel.sys;" ::: "memory");
}

__global__ void comm_pick_kernel(const unsigned long long* tables, int world, unsigned* picks_waited, unsigned timeout_ms, int* status,
                                 int* out_row) {
    __shared__ unsigned e;
    if (threadIdx.x == 0) {
        e = *picks_waited + 1u;
        *picks_waited = e;
    }
    __syncthreads();
    unsigned long long w = 0ull;
    bool arrived = true;
    if ((int)threadIdx.x < world) {
        const unsigned long long t0 = global_ns();
        const unsigned long long limit = (unsigned long long)timeout_ms * 1000000ull;
        const unsigned long long* src = tables + (e & 1u) * 8u + threadIdx.x;
        for (;;) {
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
            if ((unsigned)(w >> 48) == (e & 0xFFFFu)) break;
            if (global_ns() - t0 > limit) {
                *reinterpret_cast<volatile int*>(status) = 7;
                arrived = false;
                break;
            }
            __nanosleep(32);
        }
        w &= 0x0000FFFFFFFFFFFFull;  // value | ~row; 0 = that rank saw only NaNs
    }
    const bool all_in = __all_sync(0xffffffffu, arrived);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, w, o);
        w = other > w ? other : w;
    }
    // largest value, and among equal values the lowest row, as on one device
    if (threadIdx.x == 0) *out_row = (all_in && w) ? (int)(0xFFFFFFFFu - (unsigned)(w & 0xFFFFFFFFull)) : -1;
}

__global__ void comm_count_kernel(unsigned* counter) { *counter += 1u; }

}  // namespace

cudaError_t launch_comm_count(unsigned* counter, cudaStream_t st) {
    comm_count_kernel<<<1, 1, 0, st>>>(counter);
    return cudaGetLastError();
}

cudaError_t launch_comm_pick(const unsigned* my_flags, int world, unsigned* picks_waited, unsigned timeout_ms, int* status, bool overlap,
                             int* out_row, cudaStream_t st) {
    // `overlap` as for launch_comm_wait: this rank's own word, which its projection kernel stores
    // when its last block is done, is among the words the kernel spins on
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlap ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const unsigned long long* tables = reinterpret_cast<const unsigned long long*>(reinterpret_cast<const char*>(my_flags) + KEY_TABLE_OFFSET);
    return cudaLaunchKernelEx(&cfg, comm_pick_kernel, tables, world, picks_waited, timeout_ms, status, out_row);
}

cudaError_t launch_comm_signal(const PeerFlags& pf, unsigned* epoch_sent, cudaStream_t st) {
    comm_signal_kernel<<<1, 32, 0, st>>>(pf, epoch_sent);
    return cudaGetLastError();
}

cudaError_t launch_comm_wait(const unsigned* my_flags, int world, unsigned* epoch_waited, unsigned timeout_ms, int* status, bool overlap,
                             cudaStream_t st) {
    // With `overlap` the kernel does not wait for the grid before it (it never executes
    // griddepcontrol.wait): its own rank's flag, which that grid sets when its last block has
    // stored and fenced its outputs, is among the flags it spins on.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlap ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, comm_wait_kernel, my_flags, world, epoch_waited, timeout_ms, status);
}

}  // namespace nnb
