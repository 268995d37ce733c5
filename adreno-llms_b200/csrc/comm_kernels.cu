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

}  // namespace

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
