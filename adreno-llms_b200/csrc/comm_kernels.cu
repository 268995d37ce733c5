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

// One block per activation row m: the best (value, row) of this rank's n_local logits of that row, as the same tagged
// 64-bit word the single-token pick uses (pick number | ordered fp16 value | ~row), stored into slot [pick & 1][rank][m]
// of every rank's table.  The word is its own arrival mark.  The pick's number is one more than the counter, which the
// pick kernel (the next launch on the stream) advances when it is done.
__device__ __forceinline__ unsigned long long row_key(unsigned h, int col) {
    if ((h & 0x7FFFu) > 0x7C00u) return 0ull;  // NaNs never win
    const unsigned oh = (h & 0x8000u) ? (~h & 0xFFFFu) : (h | 0x8000u);  // order-preserving, never 0
    return ((unsigned long long)oh << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)col);
}

__global__ void __launch_bounds__(256) rows_keys_kernel(const uint16_t* __restrict__ logits, int n_local, int row_base, RowKeyTables kt,
                                                       const unsigned* __restrict__ picks_done) {
    const int m = blockIdx.x;
    const uint16_t* row = logits + (size_t)m * n_local;
    unsigned long long best = 0ull;
    // 16-byte pieces where the row allows it (eight logits per load), single values at the ragged ends
    const int head = (int)((16u - (unsigned)(reinterpret_cast<uintptr_t>(row) & 15u)) & 15u) / 2;
    const int h0 = head < n_local ? head : n_local;
    const int pieces = (n_local - h0) / 8;
    for (int i = threadIdx.x; i < h0; i += blockDim.x) {
        const unsigned long long k = row_key(row[i], row_base + i);
        best = k > best ? k : best;
    }
    const uint4* v4 = reinterpret_cast<const uint4*>(row + h0);
    for (int p = threadIdx.x; p < pieces; p += blockDim.x) {
        const uint4 v = v4[p];
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned h = (j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xFFFFu);
            const unsigned long long k = row_key(h, row_base + h0 + p * 8 + j);
            best = k > best ? k : best;
        }
    }
    for (int i = h0 + pieces * 8 + threadIdx.x; i < n_local; i += blockDim.x) {
        const unsigned long long k = row_key(row[i], row_base + i);
        best = k > best ? k : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    __shared__ unsigned long long sm[8];
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = sm[w] > best ? sm[w] : best;
        const unsigned e = *picks_done + 1u;
        // the tag is never 0, so a slot that no pick has written yet (the tables start zeroed; M may grow from call to
        // call) cannot pass for an arrived word
        const unsigned long long word = ((unsigned long long)(e % 65535u + 1u) << 48) | best;
        for (int g = 0; g < kt.world; ++g) {
            unsigned long long* dst = kt.table[g] + ((size_t)(e & 1u) * 8u + (unsigned)kt.rank) * ROW_KEYS_MAX + m;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
        }
    }
}

// One block; thread m waits (bounded) for the G words of row m that carry this pick's number and takes the largest:
// largest value, lowest row on ties, as on one device; -1 when every value of the row is NaN or a word did not arrive.
// The last thing the block does is to advance the pick counter.
__global__ void __launch_bounds__(1024) rows_pick_kernel(const unsigned long long* __restrict__ my_table, int world, int M, unsigned* picks_done,
                                                        unsigned timeout_ms, int* status, int* __restrict__ out_rows) {
    const int m = threadIdx.x;
    const unsigned e = *picks_done + 1u;
    if (m < M) {
        const unsigned long long t0 = global_ns();
        const unsigned long long limit = (unsigned long long)timeout_ms * 1000000ull;
        unsigned long long best = 0ull;
        bool arrived = true;
        for (int g = 0; g < world && arrived; ++g) {
            const unsigned long long* src = my_table + ((size_t)(e & 1u) * 8u + (unsigned)g) * ROW_KEYS_MAX + m;
            unsigned long long w;
            for (;;) {
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
                if ((unsigned)(w >> 48) == e % 65535u + 1u) break;
                if (global_ns() - t0 > limit) {
                    *reinterpret_cast<volatile int*>(status) = 7;
                    arrived = false;
                    break;
                }
                __nanosleep(32);
            }
            w &= 0x0000FFFFFFFFFFFFull;
            best = w > best ? w : best;
        }
        out_rows[m] = (arrived && best) ? (int)(0xFFFFFFFFu - (unsigned)(best & 0xFFFFFFFFull)) : -1;
    }
    __syncthreads();   // every thread has read the counter
    if (threadIdx.x == 0) *picks_done = e;
}

}  // namespace

cudaError_t launch_comm_count(unsigned* counter, cudaStream_t st) {
    comm_count_kernel<<<1, 1, 0, st>>>(counter);
    return cudaGetLastError();
}

cudaError_t launch_rows_keys(const uint16_t* logits, int M, int n_local, int row_base, const RowKeyTables& kt, const unsigned* picks_done,
                             cudaStream_t st) {
    rows_keys_kernel<<<M, 256, 0, st>>>(logits, n_local, row_base, kt, picks_done);
    return cudaGetLastError();
}

cudaError_t launch_rows_pick(const unsigned long long* my_table, int world, int M, unsigned* picks_done, unsigned timeout_ms, int* status,
                             int* out_rows, cudaStream_t st) {
    rows_pick_kernel<<<1, 1024, 0, st>>>(my_table, world, M, picks_done, timeout_ms, status, out_rows);
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
