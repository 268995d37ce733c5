// Resident decode step: data shared by the host-side plan builder (plan.cpp) and the kernel
// (decode_plan.cu).  A run of consecutive single-token operators recorded between nn_plan_begin
// and nn_plan_end becomes ONE launch whose blocks stay on their multiprocessors and walk a table
// of operator descriptors: the role of the reference's recordable-queue replay
// (src/models/smollm2-135m-instruct/src/model.cpp:104-195,312-344), which exists to take the
// per-dispatch cost out of the decode loop.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "kernels.h"

namespace nnb {

// One weight of an operator (fused QKV has three).
struct PlanSeg {
    const uint16_t* scale;        // int8: [N] row scales (Q4 block scales travel by tensor copy); null for fp16
    uint16_t* out;                // fp16 destination; null when a later operator of the run overwrites these values
    unsigned long long* ll_out;   // published copy for readers inside the run, or null when there is none:
                                  // word j = fp16 of row 2j | fp16 of row 2j+1 << 16 | epoch << 32
    int N;                        // rows
    int tile0;                    // first tile of this weight inside the operator
};

// The scalar half of a descriptor (copied to shared memory by the consumers, 16 x 16 bytes).
struct PlanOpScalars {
    PlanSeg seg[3];
    const uint16_t* scale2;              // two-weight epilogue: scales of the "up" weight
    const uint16_t* x;                   // activations [K] fp16 written before the run started, or null
    const unsigned long long* x_ll;      // ... or the published output of an earlier operator of the run
    const uint16_t* res;                 // in-place epilogues: the previous values when written before the run, or null
    const unsigned long long* res_ll;    // ... or the published output of an earlier operator of the run
    const uint16_t* norm_w;              // RMSNorm prologue weight [K] fp16, or null
    unsigned long long* argmax_slot;     // fused greedy pick (kernels.h: LinArgs), or null
    unsigned* argmax_done;
    int* argmax_out;
    float norm_eps;
    int argmax_base;
    int fmt, epi, dual, ksplit;
    int kcb, nchunks, groups, rowbytes;
    int K, nseg, ntiles, tile_start;     // tile_start: tiles of the run before this operator, modulo the grid
    int item_bytes, nbox, flags;         // flags: PLAN_EVICT_FIRST | PLAN_SCALE_TMA | PLAN_ROW_SCALES
    int scale_off;                       // int8 row scales ride in the last item of each tile, at this offset inside it
    int x_epoch, res_epoch, epoch, nblocks;  // epochs are 1 + index of the producing operator; nblocks = blocks that hold tiles of this one
};
static_assert(sizeof(PlanOpScalars) == 256, "descriptor scalars are copied in sixteen 16-byte pieces");

struct alignas(128) PlanOp {
    CUtensorMap tm[4];    // weight views: seg[0..2], and the second weight of the two-weight epilogue
    CUtensorMap tm_s[4];  // Q4 block-scale views, same order
    PlanOpScalars s;
};

enum : int {
    PLAN_EVICT_FIRST = 1,  // weights larger than L2 are streamed with an evict-first policy
    PLAN_SCALE_TMA = 2,    // Q4: block scales arrive by tensor copies
    PLAN_ROW_SCALES = 4,   // int8: the tile's row scales arrive with its last item (bulk copy), when the tile's rows allow it
    PLAN_BIAS = 8,         // a bias row per segment is added to the stored result (PlanParams::bias)
};
constexpr int PLAN_ROW_SCALE_BYTES = 1024;  // room for them at the end of an item: first weight at +0, second at +512
// Bulk copies move multiples of 16 bytes: a tile's row scales travel with it when its valid rows are a multiple of 8.
__host__ __device__ inline bool plan_rows_bulk_ok(int rows_valid) { return rows_valid > 0 && (rows_valid & 7) == 0; }

constexpr int PLAN_SLOTS = 16;        // ring items in flight per block
constexpr int PLAN_MAX_OPS = 1024;    // operators per run (their tile table sits in shared memory)
// head of the kernel's shared memory: 64 bytes of zeros, full[] and empty[] barriers, the producer's
// table of items in flight (offset and end of each), the count of items issued by a producer that stopped early
constexpr int PLAN_HDR_BARS = 64;
constexpr int PLAN_HDR_SLOTS = PLAN_HDR_BARS + 2 * PLAN_SLOTS * 8;
constexpr int PLAN_HDR_ISSUED = PLAN_HDR_SLOTS + 2 * PLAN_SLOTS * 4;
constexpr int PLAN_HDR_STATE = PLAN_HDR_ISSUED + 16;  // the consumers' state between operators (64 bytes)
constexpr int PLAN_HDR_BYTES = 640;
static_assert(PLAN_HDR_STATE + 64 <= PLAN_HDR_BYTES, "header layout");

struct PlanParams {
    const PlanOp* ops;
    const int2* op_tiles;   // per operator: (tile_start modulo grid, tiles)
    int nops;
    unsigned* state;        // [0] launches completed, [1] blocks finished (returns to 0), [2] abort flag (returns to 0)
    int* status;            // mapped host word: non-zero when a bounded wait ran out
    long long wait_cycles;  // limit of every wait
    int drop_publish_op;    // fault injection for tests: this operator never publishes its outputs (-1: none)
    const uint16_t* const* bias;  // [nops][3] bias rows of the operators flagged PLAN_BIAS (null when the run has none)
    int off_tiles, off_desc, off_xraw, off_xs, off_ctab, off_norm, off_gamma, off_red, off_ring, ring_bytes;
};

// decode_plan.cu
cudaError_t decode_plan_configure();
cudaError_t decode_plan_func(const void** func);   // the kernel's address, for a graph kernel node
constexpr int DECODE_PLAN_THREADS = (8 + 1) * 32;  // eight consumer warps (one per K part of a split tile) and the producer warp

// ---- host side (plan.cpp) ---------------------------------------------------------------------
// What the recorder keeps of one streamed single-token operator.
struct RecordedOp {
    int fmt;
    LinArgs a;       // complete arguments, as launch_stream received them
    StreamPlan p;    // geometry chosen for the separate launch (the resident kernel keeps its K partition)
    cudaGraphNode_t node;  // the captured kernel node
    bool eligible;   // the resident kernel can run it
};

// Data hazards between the operators of a candidate run, resolved at record time.
struct OpDeps {
    int x_dep = -1, x_dep_seg = 0;      // operator (and weight) whose output is this operator's x; -1: written before the run
    int res_dep = -1, res_dep_seg = 0;  // same for the values an in-place epilogue updates
    bool store[3] = {true, true, true};       // false: a later operator of the run overwrites this output
    bool publish[3] = {false, false, false};  // an operator of the run reads this output
};
struct HazardOp {  // address ranges only; kept separate from LinArgs so that the analysis is testable on its own
    uintptr_t x = 0; size_t x_bytes = 0;
    int nout = 0;
    uintptr_t out[4] = {0, 0, 0, 0}; size_t out_bytes[4] = {0, 0, 0, 0};  // weights' outputs, then (optionally) the arg-max index
    bool inplace = false;    // reads out[0] before writing it
    bool has_argmax = false;
};
// Longest prefix of ops[first..] that can run as one resident launch: every read of a value produced
// inside the prefix names its producer exactly (same address range), and every overwrite is ordered
// behind the reads and writes it must follow by the activations' own data flow.  Fills deps[0..len).
int analyze_run(const std::vector<HazardOp>& ops, int first, std::vector<OpDeps>* deps);

struct PlanRun {
    int first = 0, count = 0;        // recorded operators [first, first + count)
    PlanOp* d_ops = nullptr;
    int2* d_tiles = nullptr;
    unsigned long long* d_ll = nullptr;
    const uint16_t** d_bias = nullptr;
    unsigned* d_state = nullptr;
    PlanParams params = {};
    int grid = 0;
    size_t smem = 0;
};
// Builds the device tables of one run.  Returns cudaSuccess and fills `run`, or an error (the caller
// then keeps the separate launches).  `reason` receives a short text when the run cannot be built.
cudaError_t build_run(const std::vector<RecordedOp>& rec, const std::vector<OpDeps>& deps, int first, int count, int sm_count, size_t smem_limit,
                      int* status_dev, PlanRun* run, const char** reason);
void free_run(PlanRun* run);

// gemv_stream.cu: tensor maps of a streamed operator (weights: 128-byte swizzled boxes of `box_rows`
// rows; Q4 scales: dense boxes of `box_bytes` x `box_rows`).
bool make_weight_map(CUtensorMap* m, const void* W, int rows, int rowbytes, int box_rows);
bool make_scale_map(CUtensorMap* m, const void* S, int rows, int rowbytes, int box_bytes, int box_rows);

}  // namespace nnb
