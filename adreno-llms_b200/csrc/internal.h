// Internal state shared by the C-ABI translation units (not installed).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "plan.h"

struct QuantEntry {
    int fmt;
    const uint16_t* scale;
    int N, K;
    size_t rowbytes;
    // Q4 whose scale rows (K / 16 bytes) are not a multiple of 16 bytes: a copy of the scales with the rows padded to
    // one, owned by the library, so that tensor copies can fetch them (the weights themselves are never repacked)
    uint16_t* scale_pad = nullptr;
    int scale_pitch = 0;  // bytes
};
inline void free_scale_pad(QuantEntry& q) {
    if (q.scale_pad) cudaFree(q.scale_pad);
    q.scale_pad = nullptr;
}

// Per-launch profile behind the reference's switches NNOPT_KERNEL_PROFILE / NNOPT_PROFILE
// (src/models/lfm2-5-350m/src/kernel_profiler.cpp:18-62, src/models/smollm2-135m-instruct/src/prof.cpp:36-131):
// a CUDA event pair around every call, aggregated by label at nn_shutdown or nn_profile_report.
struct ProfPending {
    std::string label;
    cudaEvent_t start, stop;
};
struct ProfAgg {
    unsigned long long count = 0;
    double total_us = 0, max_us = 0;
};

struct nn_context {
    int device = 0;
    int sm_count = 0;
    size_t l2_bytes = 0, hbm_bytes = 0, smem_limit = 0;
    cudaStream_t stream = nullptr;
    std::map<uintptr_t, QuantEntry> registry;  // keyed by weight device pointer
    int* status_host = nullptr;                // mapped pinned word written by kernels
    int* status_dev = nullptr;
    unsigned long long* argmax_slot = nullptr;
    void* stage_img = nullptr;      // staged activations of a batched call, written once per launch (stage_image.cu)
    size_t stage_img_bytes = 0;
    void* pair_scratch = nullptr;   // fp16 results of the two projections of a two-weight form at prefill row counts
    size_t pair_scratch_bytes = 0;
    void* norm_scratch = nullptr;   // normalised activations when the fused prologue does not apply
    size_t norm_scratch_bytes = 0;
    float* sk_scratch = nullptr;   // partial sums of blocks that share a tile (balanced K-streaming)
    unsigned* sk_flags = nullptr;
    void* flush_buf = nullptr;
    size_t flush_bytes = 0;
    bool use_pdl = true;
    bool capturing = false;
    std::vector<nnb::RecordedOp> rec;  // streamed single-token operators of the recording in progress
    bool profiling = false;
    std::vector<ProfPending> prof_pending;
    std::map<std::string, ProfAgg> prof;
    long long launches = 0, launches_at_capture = 0;
};

namespace nnb {

struct ResolvedW {
    int fmt;
    const uint16_t* scale;
    int rows_avail;  // -1 when W is not a registered weight (fp16)
    const uint16_t* scale_pad;  // the padded copy of the Q4 scales from the view's first row on, or null
    int scale_pitch;
};
bool resolve_weight(const nn_context* c, const void* W, int K, ResolvedW* out);

// nn_linear that also stores every output at the same offset of `npeer` peer-mapped buffers and,
// with `sig`, sends the gather's completion signal from the (last) kernel itself; api.cpp
struct GatherSignal;
int linear_to_peers(nn_context* c, int M, int N, int K, void* x, void* W, void* out, uint16_t* const* peers, int npeer,
                    const GatherSignal* sig, const char* who);

// nn_linear_argmax with the winning row reported as row_base + row; with `sig` the kernel leaves
// its best key in every rank's key table and sends the completion signal instead of writing
// out_idx (the wait kernel that follows picks among the ranks); api.cpp
int linear_argmax(nn_context* c, int N, int K, void* x, void* W, void* logits, void* out_idx, int row_base, const GatherSignal* sig,
                  const char* who);

int fail(int code, const char* file, int line, const char* fmt, ...) __attribute__((format(printf, 4, 5)));

}  // namespace nnb

#define NN_FAIL(code, ...) nnb::fail((code), __FILE__, __LINE__, __VA_ARGS__)
