// Internal launch interface between the C-ABI layer (api.cpp) and the CUDA
// translation units.  Nothing here is exported from the shared library.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace nnb {

enum Fmt : int { FMT_FP16 = 0, FMT_INT8 = 1, FMT_Q4 = 2 };

// What work-item 0 of the reference kernels does with the reduced sum.
enum Epi : int {
    EPI_STORE = 0,      // out = half(acc)
    EPI_RESIDUAL = 1,   // out = half(float(out) + acc)               (in place)
    EPI_SWIGLU = 2,     // out = half(silu(acc_gate) * acc_up)        (two weights)
    EPI_SILU_GATE = 3,  // out = half(out * sigmoid(out) * acc)       (in place)
};

// Byte offset, inside each rank's symmetric flag allocation, of the key tables of the row-sharded
// greedy pick: two tables (parity of the pick number) of eight 64-bit words, word g written by
// rank g: pick number (16 bits) | ordered fp16 value (16 bits) | ~row (32 bits).
constexpr int KEY_TABLE_OFFSET = 64;

// Completion signal of a row-sharded gather, sent by the projection kernel itself: the last
// block to finish publishes the next epoch number in word `rank` of every rank's flag array.
struct GatherSignal {
    unsigned* flags[8];  // flags[g] = rank g's flag array (peer-mapped for g != rank)
    unsigned* epoch;     // local: signals sent so far (with a fused arg-max: picks sent so far)
    unsigned* done;      // local: blocks of the current launch that have finished (returns to 0);
                         // unused with a fused arg-max, whose key word is its own arrival mark
    int world, rank;     // world == 0: no signal
};

struct LinSeg {
    const uint8_t* W;       // [N, rowbytes] row-major, on-disk layout
    const uint16_t* scale;  // int8: [N]; Q4: [N, K/32]; fp16: null
    uint16_t* out;          // [M, ld_out] fp16 (or the in/out vector)
    int N;                  // rows of this segment
    int ld_out;             // leading dimension of out (elements)
    int tile0;              // first 32-row tile of this segment in the launch
    // optional bias row (fp16 [N]) added to the stored result the way the reference's bias kernel does it after the
    // projection: out = half(float(half(sum)) + float(bias[n])) (bias_add_rowmajor, src/models/qwen2-5-0-5b/kernels/bias_add.cl:18-40)
    const uint16_t* bias;
};

struct LinArgs {
    LinSeg seg[3];  // up to three weights sharing x (fused QKV); normally one
    int nseg;
    const uint8_t* W2;       // EPI_SWIGLU: the "up" weight (seg[0] is the gate)
    const uint16_t* scale2;  // EPI_SWIGLU: its scales
    const uint16_t* x;       // [M, K] fp16
    int M, K;
    int ntiles;      // row tiles over all segments
    int epi;         // Epi
    int kcb;         // bytes of one weight row moved per pipeline stage
    int kw;          // warps that split K of one tile (1, 2 or 4)
    int* status;     // device word: non-zero when a bounded wait ran out
    // optional fused arg-max over the fp16 values of seg[0] (M == 1, one segment): every block
    // folds its rows into argmax_slot (packed ordered value << 32 | ~index, atomicMax, 0 before
    // and after the launch); the block that finishes last writes the index and clears the words.
    // seg[0].out may then be null (the logits are not stored).
    unsigned long long* argmax_slot;
    unsigned* argmax_done;   // blocks finished (returns to 0)
    int* argmax_out;         // device int: winning row + argmax_base, -1 when every value is NaN
    int argmax_base;
    // row-sharded gather: the same block of seg[0].out in the other ranks' gather buffers
    // (peer-mapped device pointers); every stored value is also written there
    uint16_t* peer_out[7];
    int npeer;
    GatherSignal sig;
    // balanced K-streaming: block b takes pipeline items [b T / G, (b+1) T / G) of the launch's
    // T = tiles x K-groups items, so a tile may be shared by neighbouring blocks; the block that
    // holds the head of a tile adds the others' fp32 partial sums (fixed order) and stores it
    // optional RMSNorm of the activations before the projection (fused prologue):
    // x_used[m][k] = half((x[m][k] * rsqrt(mean_k x[m]^2 + eps)) * norm_w[k])
    const uint16_t* norm_w;  // fp16 [K], null = no norm
    float norm_eps;
    // batched calls (M >= 2): the staged form of the activations, written once per launch by
    // stage_image_kernel in the kernel's own shared-memory layout; every block copies it in
    const uint8_t* staged;
    unsigned staged_bytes;
    // host side only: Q4 scales with rows padded to a multiple of 16 bytes (seg[0..2], then the second weight of the
    // two-weight form), for the tensor copies when K / 16 is not such a multiple; all null otherwise
    const uint16_t* scale_pad[4];
    int scale_pitch;
    float* sk_scratch;    // [blocks][consumer threads][2 * NT * 4] partial sums
    unsigned* sk_flags;   // [blocks] "partial written", consumed and cleared by the tile's owner
    int streamk;
};

struct StreamPlan {  // launch geometry chosen on the host
    int grid;
    int kcb;     // bytes of one weight row per pipeline stage
    int kw;      // warps splitting K of one tile
    int warps;   // warps per block
    int stages;  // ring depth
    int ntiles;  // block tiles over all segments
    size_t smem;
    bool ok;
    bool streamk;  // items are dealt out evenly across the grid instead of whole tiles
};

// gemv_stream.cu
constexpr int SK_MAX_BLOCKS = 1024;                         // grid limit of a balanced launch (sizes its scratch)
constexpr size_t SK_SCRATCH_BYTES = (size_t)SK_MAX_BLOCKS * 128 * 16 * sizeof(float);
bool stream_supported(int fmt, int M, int K, const LinArgs& a);
StreamPlan stream_plan(int fmt, const LinArgs& a, int sm_count, size_t smem_limit);
cudaError_t launch_stream(int fmt, const LinArgs& a, const StreamPlan& p, cudaStream_t st, bool pdl);
cudaError_t stream_configure();  // opt in to large dynamic shared memory, once per device

// 2-D tensor map helper (gemv_stream.cu): [dim1][dim0] elements, row stride in bytes, box dim0 x dim1,
// 128-byte swizzle (or none); fp16 elements when `half_elems`, bytes otherwise.
bool encode_tiled_2d(void* map, bool half_elems, const void* base, uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes,
                     uint32_t box0, uint32_t box1, bool swizzle128 = true);

// gemm_tc.cu: tcgen05 / tensor-memory GEMM for M > 16
cudaError_t gemm_tc_configure();
bool gemm_tc_supported(int fmt, int M, int N, int K, const void* x, const void* W, const void* out);
// W in its registered format; scale = int8 row scales / Q4 block scales / null
cudaError_t launch_gemm_tc(int fmt, const void* W, const uint16_t* scale, const uint16_t* x, uint16_t* out, int M, int N, int K,
                           int ld_out, int epi, int* status, uint16_t* const* peer_out, int npeer, const GatherSignal* sig, cudaStream_t st);

// gemv_generic.cu: any K, any alignment (the reference's gemv_rT_fp32acc role)
cudaError_t launch_generic(int fmt, const LinArgs& a, cudaStream_t st);

// comm_kernels.cu: cross-rank flags in peer-mapped memory
struct PeerFlags {
    unsigned* flags[8];  // flags[g] = base of rank g's flag array (peer-mapped for g != rank)
    int world, rank;
};
cudaError_t launch_comm_signal(const PeerFlags& pf, unsigned* epoch_sent, cudaStream_t st);
// `overlap`: launch with programmatic stream serialisation so that the wait starts spinning while
// the kernel before it still runs (valid when that kernel sends this rank's own signal).
cudaError_t launch_comm_wait(const unsigned* my_flags, int world, unsigned* epoch_waited, unsigned timeout_ms, int* status, bool overlap,
                             cudaStream_t st);
// Row-sharded greedy pick: waits (bounded) for pick number *picks_waited + 1 of every rank in this
// rank's key tables and writes the winning row (-1: every value was NaN, or the wait ran out).
cudaError_t launch_comm_count(unsigned* counter, cudaStream_t st);
// Row-sharded greedy pick of M rows at once.  Key tables: [2][8 ranks][ROW_KEYS_MAX] 64-bit words on every rank.
constexpr int ROW_KEYS_MAX = 1024;
constexpr size_t ROW_KEYS_BYTES = (size_t)2 * 8 * ROW_KEYS_MAX * 8;
struct RowKeyTables { unsigned long long* table[8]; int world, rank; };
cudaError_t launch_rows_keys(const uint16_t* logits, int M, int n_local, int row_base, const RowKeyTables& kt, const unsigned* picks_done,
                             cudaStream_t st);
cudaError_t launch_rows_pick(const unsigned long long* my_table, int world, int M, unsigned* picks_done, unsigned timeout_ms, int* status,
                             int* out_rows, cudaStream_t st);
cudaError_t launch_comm_pick(const unsigned* my_flags, int world, unsigned* picks_waited, unsigned timeout_ms, int* status, bool overlap,
                             int* out_row, cudaStream_t st);

// misc.cu
// Multiprocessors of the current device (cached per device; allocates nothing).
int current_sm_count();
cudaError_t launch_dequant(int fmt, int N, int K, const void* W, const uint16_t* scale, float* out, cudaStream_t st);
cudaError_t launch_argmax_half(const uint16_t* v, int n, int* out_idx, unsigned long long* slot, cudaStream_t st);
cudaError_t launch_fill_u64(unsigned long long* p, unsigned long long v, cudaStream_t st);
cudaError_t launch_argmax_finish(const unsigned long long* slot, int* out_idx, cudaStream_t st);
// Q4 block scales by tensor copy: from the weight's own scale array when its rows (K / 16 bytes) are a multiple of 16 bytes
// and 16-byte aligned, else from the padded copy made at registration.  False: neither is there (per-lane copies then).
inline bool q4_scale_views(const LinArgs& a, const uint16_t* base[4], int* pitch) {
    const bool dual = a.epi == EPI_SWIGLU;
    bool nat = a.K % 256 == 0, pad = a.scale_pitch > 0;
    for (int i = 0; i < a.nseg; ++i) {
        nat = nat && (reinterpret_cast<uintptr_t>(a.seg[i].scale) & 15) == 0;
        pad = pad && a.scale_pad[i] != nullptr;
    }
    if (dual) {
        nat = nat && (reinterpret_cast<uintptr_t>(a.scale2) & 15) == 0;
        pad = pad && a.scale_pad[3] != nullptr;
    }
    if (!nat && !pad) return false;
    for (int i = 0; i < 3; ++i) base[i] = nat ? a.seg[i].scale : a.scale_pad[i];
    base[3] = nat ? a.scale2 : a.scale_pad[3];
    *pitch = nat ? a.K / 16 : a.scale_pitch;
    return true;
}
cudaError_t launch_l2_flush(void* buf, size_t bytes, cudaStream_t st);
cudaError_t launch_silu_mul(const uint16_t* g, const uint16_t* u, uint16_t* out, size_t n, cudaStream_t st);
// the staged activations of a batched call (layout of the streaming kernel's shared memory), with the optional RMSNorm
size_t stage_image_bytes(int fmt, int M, int K);
cudaError_t launch_stage_image(int fmt, const uint16_t* x, int M, int K, const uint16_t* norm_w, float eps, uint8_t* img, cudaStream_t st,
                               bool pdl);
// read-bandwidth probes over `bytes` (a multiple of 16 KiB) at src; sink: 256 floats; status: one word, set on a timed-out wait
cudaError_t launch_probe_loads(const void* src, size_t bytes, float* sink, cudaStream_t st);
cudaError_t launch_probe_tma(const void* src, size_t bytes, unsigned* status, cudaStream_t st);
struct BiasArgs {  // up to three [rows, cols] fp16 outputs with a bias row each
    uint16_t* out[3];
    const uint16_t* bias[3];
    int cols[3];
    int rows, nseg;
};
cudaError_t launch_bias_add(const BiasArgs& a, cudaStream_t st);
cudaError_t launch_rmsnorm(const uint16_t* x, const uint16_t* w, uint16_t* out, int rows, int cols, float eps, cudaStream_t st);

}  // namespace nnb
