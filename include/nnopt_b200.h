/*
 * nnopt_b200 — C ABI of the B200 (sm_100a) replacement for the decode-time
 * linear operators of a8nova/adreno-llms.
 *
 * The library replaces the reference's OpenCL buffer + kernel dispatch for ONE
 * path: out[M,N] = x[M,K] . W[N,K]^T with W stored as fp16, per-row symmetric
 * int8 (+ fp16 scale per row) or packed 4-bit (+ fp16 scale per 32 weights),
 * plus the fused epilogues the reference's layers call at decode time.
 * Each entry point names the reference interface it stands in for
 * (paths relative to the reference project).
 *
 * Conventions
 *   - nn_buf is a CUDA device pointer (the role cl_mem plays in the reference).
 *     The library never frees caller buffers.  Activations, scales and outputs
 *     are IEEE binary16; weights keep the exact on-disk byte layout written by
 *     scripts/convert_hf_to_bin.py and src/models/<model>/scripts/quantize_*.py.
 *   - Every call is asynchronous on the context's single stream (the role of the
 *     reference's one in-order cl_command_queue): a result is visible to the next
 *     call on the same context without a host sync (nn_sync to wait on the host).
 *   - One host thread per context; contexts are independent (one per GPU).
 *   - Returns 0 (NN_OK) or a negative code; nn_last_error() gives the text
 *     (thread-local).  Nothing aborts or throws across this boundary.  There is
 *     no CPU fallback: without a CUDA device nn_init fails.
 */
#ifndef NNOPT_B200_H
#define NNOPT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nn_context nn_context; /* OpenCLContext + its cl_command_queue */
typedef struct nn_weights nn_weights; /* class Weights */
typedef struct nn_plan nn_plan;       /* a recorded decode step */
typedef struct nn_comm nn_comm;       /* row-sharding communicator (one rank per GPU) */
typedef void* nn_buf;                 /* device pointer; stands in for cl_mem */

enum {
    NN_OK = 0,
    NN_ERR_ARG = -1,         /* bad argument (null buffer, shape/registration mismatch) */
    NN_ERR_CUDA = -2,        /* a CUDA runtime call failed */
    NN_ERR_UNSUPPORTED = -3, /* shape or mode not handled by any kernel */
    NN_ERR_IO = -4,          /* weight bundle could not be read or parsed */
    NN_ERR_NOTFOUND = -5,    /* tensor key missing */
    NN_ERR_COMM = -6,        /* NCCL missing or a collective failed */
    NN_ERR_TIMEOUT = -7      /* a bounded device-side wait ran out */
};

const char* nn_last_error(void);
const char* nn_version(void);

/* ---- context: src/models/smollm2-135m-instruct/src/opencl_context.cpp:171-205
 *      (OpenCLContext::initialize, one device, one in-order queue) ------------- */
int nn_init(int device_ordinal, nn_context** out_ctx);
int nn_shutdown(nn_context* ctx); /* frees registry entries and library-owned buffers */
void* nn_stream(nn_context* ctx); /* the cudaStream_t every call is ordered on */
int nn_sync(nn_context* ctx);     /* host wait; also reports a recorded device-side timeout */
int nn_device_info(nn_context* ctx, int* sm_count, size_t* l2_bytes, size_t* hbm_bytes);

/* ---- buffers: clCreateBuffer / clEnqueueWriteBuffer / clEnqueueReadBuffer /
 *      clReleaseMemObject as used by src/models/lfm2-5-350m/src/weights.cpp:286-291
 *      and the layers' persistent activation buffers ----------------------------- */
nn_buf nn_buf_alloc(nn_context* ctx, size_t bytes); /* NULL on failure */
int nn_buf_free(nn_context* ctx, nn_buf buf);
int nn_buf_write(nn_context* ctx, nn_buf dst, size_t dst_offset, const void* src, size_t bytes); /* H2D, async */
int nn_buf_read(nn_context* ctx, void* dst, nn_buf src, size_t src_offset, size_t bytes);        /* D2H, async */
int nn_buf_copy(nn_context* ctx, nn_buf dst, nn_buf src, size_t bytes);                          /* D2D, async */
int nn_buf_fill(nn_context* ctx, nn_buf dst, int byte_value, size_t bytes);
void* nn_host_alloc(size_t bytes); /* pinned host memory for nn_buf_write / nn_buf_read */
int nn_host_free(void* p);

/* ---- quantised-weight registry: nnopt_register_int8_weight /
 *      nnopt_register_q4_weight, src/models/lfm2-5-350m/src/utils.h:127,132
 *      (utils.cpp:357-368, 584-595).  Keyed by the weight's device pointer; a
 *      row-range sub-view W + r*rowbytes of a registered weight resolves too (the
 *      reference's row tiles, utils.cpp:427-452).  The weights are never repacked.  Register
 *      after the weight and its scales have been written: for a Q4 weight whose scale rows
 *      (K / 16 bytes) are not a multiple of 16 bytes the library keeps its own copy of the
 *      scales with the rows padded to one (N * roundup(K / 16, 16) bytes, freed when the
 *      weight is unregistered or freed), taken at registration on the context's stream. --- */
int nn_register_int8_weight(nn_context* ctx, nn_buf W_int8, nn_buf scale_fp16, int N, int K);
int nn_register_q4_weight(nn_context* ctx, nn_buf W_q4, nn_buf scale_fp16, int N, int K_unpacked);
int nn_unregister_weight(nn_context* ctx, nn_buf W);

/* ---- the operator: pytorch_linear(queue, M, N, K, x, W, out),
 *      src/models/lfm2-5-350m/src/utils.h:117-119 (utils.cpp:1263-1374);
 *      same call in src/models/qwen2-5-0-5b/src/utils.cpp:758-826 and
 *      src/models/smollm2-135m-instruct/src/utils.cpp:279-340.
 *      out[M,N] = x[M,K] . W[N,K]^T.  Format is picked by registry lookup on W in
 *      the reference's order: Q4, then int8, else fp16.  M > 1 is M independent
 *      M = 1 results (the reference loops M = 1 for quantised weights,
 *      src/models/lfm2-5-350m/src/model.cpp:243-251). ----------------------------- */
int nn_linear(nn_context* ctx, int M, int N, int K, nn_buf x, nn_buf W, nn_buf out);

/* residual[M,N] = half(float(residual) + x.W^T), in place: Qwen's
 * pytorch_linear_add (src/models/qwen2-5-0-5b/src/utils.cpp:862-882) and SmolLM2's
 * fused_oproj_residual / fused_down_residual kernels
 * (src/models/smollm2-135m-instruct/kernels/block_fused_int8.cl:105,238;
 *  host: src/layers/attention.cpp:771-806, src/layers/mlp.cpp:340-373). */
int nn_linear_add(nn_context* ctx, int M, int N, int K, nn_buf x, nn_buf W, nn_buf residual_inout);

/* gate_inout[n] = half(gate * sigmoid(gate) * (W3.x)[n]): pytorch_linear_silu_gate_fused,
 * src/models/lfm2-5-350m/src/utils.h:140-142 (utils.cpp:1377-1406, kernels/mlp_fused.cl:19-73).
 * The reference form is M = 1; M rows are accepted here. */
int nn_linear_silu_gate_fused(nn_context* ctx, int M, int N, int K, nn_buf x, nn_buf W3, nn_buf gate_inout);

/* out[M,N] = half(silu(x.Wg^T) * (x.Wu^T)): fused_gate_up_silu_m1,
 * src/models/qwen2-5-0-5b/src/utils.cpp:478-487 and
 * src/models/smollm2-135m-instruct/kernels/block_fused.cl:334,475,533 /
 * block_fused_int8.cl:176-231 (host: src/layers/mlp.cpp:298-337).
 * Wg and Wu must be of the same format. */
int nn_fused_gate_up_silu(nn_context* ctx, int M, int N, int K, nn_buf x, nn_buf Wg, nn_buf Wu, nn_buf out);

/* Three projections of the same x in one launch: fused_qkv_gemv_m1,
 * src/models/smollm2-135m-instruct/kernels/block_fused.cl:192 (host:
 * src/layers/attention.cpp:653-722).  q[M,Nq], k[M,Nk], v[M,Nv]; same format. */
int nn_linear_qkv(nn_context* ctx, int M, int K, nn_buf x, nn_buf Wq, int Nq, nn_buf Wk, int Nk, nn_buf Wv, int Nv,
                  nn_buf q, nn_buf k, nn_buf v);

/* The same with Qwen's q/k/v bias added afterwards, and the bias add on its own:
 * bias_add_rowmajor, src/models/qwen2-5-0-5b/kernels/bias_add.cl:18-40 (host:
 * src/layers/attention.cpp:413-469): out[r,c] = half(float(out[r,c]) + float(bias[c])), applied to
 * the fp16 result of the projection, as the reference does: same bits as nn_linear_qkv followed by
 * nn_bias_add.  Up to 16 rows the bias is part of the projection's epilogue (no launch of its own,
 * and the call can join a resident run of a recorded step); above, one bias launch follows. */
int nn_linear_qkv_bias(nn_context* ctx, int M, int K, nn_buf x, nn_buf Wq, int Nq, nn_buf Wk, int Nk, nn_buf Wv, int Nv,
                       nn_buf bias_q, nn_buf bias_k, nn_buf bias_v, nn_buf q, nn_buf k, nn_buf v);
int nn_bias_add(nn_context* ctx, int rows, int cols, nn_buf out_inout, nn_buf bias_fp16);

/* RMSNorm on fp16 storage: out[r,c] = half( (x[r,c] * rsqrt(mean_c x[r,c]^2 + eps)) * weight[c] )
 * (rmsnorm_forward, src/models/smollm2-135m-instruct/kernels/rmsnorm.cl:27-104; host
 * src/layers/layer_norm.cpp:76-126).  The three nn_rmsnorm_* forms below are nn_linear,
 * nn_linear_qkv and nn_fused_gate_up_silu applied to that normalised row, the pairs
 * input_layernorm -> QKV and post_attention_layernorm -> gate/up of a decoder layer: for
 * M <= 16 the norm is the prologue of the projection kernel (no launch, no round trip of the
 * normalised row through memory); otherwise it runs as a launch of its own into context scratch
 * (which can only grow outside a recording). */
int nn_rmsnorm(nn_context* ctx, int rows, int cols, nn_buf x, nn_buf weight_fp16, float eps, nn_buf out);
int nn_rmsnorm_linear(nn_context* ctx, int M, int N, int K, nn_buf x, nn_buf norm_weight, float eps, nn_buf W, nn_buf out);
int nn_rmsnorm_linear_qkv(nn_context* ctx, int M, int K, nn_buf x, nn_buf norm_weight, float eps, nn_buf Wq, int Nq, nn_buf Wk, int Nk,
                          nn_buf Wv, int Nv, nn_buf q, nn_buf k, nn_buf v);
/* ... and with Qwen's q/k/v bias (input_layernorm -> q/k/v projections -> bias_add_rowmajor,
 * src/models/qwen2-5-0-5b/src/layers/attention.cpp:303-317,413-469) in the same call. */
int nn_rmsnorm_linear_qkv_bias(nn_context* ctx, int M, int K, nn_buf x, nn_buf norm_weight, float eps, nn_buf Wq, int Nq, nn_buf Wk, int Nk,
                               nn_buf Wv, int Nv, nn_buf bias_q, nn_buf bias_k, nn_buf bias_v, nn_buf q, nn_buf k, nn_buf v);
int nn_rmsnorm_gate_up_silu(nn_context* ctx, int M, int N, int K, nn_buf x, nn_buf norm_weight, float eps, nn_buf Wg, nn_buf Wu, nn_buf out);

/* fp32 [N,K] = the dequantised weight exactly as the kernels unpack it
 * (src/models/lfm2-5-350m/kernels/gemv_m1_q4.cl:31-40; scripts/quantize_q4.py:156-166;
 *  scripts/quantize_weights.py:135-139).  For bit-exact checks of the unpack rule. */
int nn_dequant(nn_context* ctx, int N, int K, nn_buf W, nn_buf out_f32);

/* index of the largest fp16 logit (lowest index on ties) into a device int:
 * argmax_block + argmax_final, src/models/lfm2-5-350m/kernels/argmax.cl:30,90
 * (host: src/model.cpp:603-623). */
int nn_argmax(nn_context* ctx, int n, nn_buf logits_fp16, nn_buf out_index_i32);

/* lm_head and greedy pick in one launch (M = 1): out_index = arg-max over n of
 * fp16( x[K] . W[n,K] ), the index nn_linear followed by nn_argmax would give.  `logits_fp16`
 * may be NULL, in which case the N logits are never written (the reference's profile names the
 * logits write as the lm_head's bottleneck, src/models/smollm2-135m-instruct/BENCHMARK.md:549-551).
 * Replaces the pair LmHead::forward + argmax_block/argmax_final
 * (src/models/smollm2-135m-instruct/src/layers/lm_head.cpp:36-67, kernels/argmax.cl:33,80). */
int nn_linear_argmax(nn_context* ctx, int N, int K, nn_buf x, nn_buf W, nn_buf logits_fp16, nn_buf out_index_i32);

/* Arg-max for callers that are not allowed to allocate device memory (a real-time thread
 * under a no-allocation rule, a host application that owns the whole device heap through its
 * own pool, a service whose memory budget is frozen after start-up).  It has no counterpart
 * in the reference; it is nn_argmax without a context: the reduction scratch is a fixed
 * array inside the library image on every GPU that loads it (256 bytes), so nothing is ever
 * allocated or freed.  `cuda_stream` is the cudaStream_t to order the work on (NULL = the
 * default stream); the current device is used.
 *   - n must be <= NN_ARGMAX_STATIC_MAX_N, otherwise NN_ERR_ARG.
 *   - The first call on each device resolves the scratch array's device address; make that
 *     first call before any stream capture.
 *   - All calls on a device share the scratch.  Each call clears what it uses first, so
 *     results never depend on earlier calls, but calls that overlap on the GPU race;
 *     order them on one stream. */
#define NN_ARGMAX_STATIC_MAX_N (1 << 22)
int nn_argmax_static(void* cuda_stream, int n, nn_buf logits_fp16, nn_buf out_index_i32);

/* ---- recorded decode step: the reference's recordable-queue replay
 *      (src/models/smollm2-135m-instruct/src/model.cpp:104-195,312-344;
 *      src/models/lfm2-5-350m/src/model.cpp:188-228,376-458).
 *      Between nn_plan_begin and nn_plan_end the operator calls above (and anything else the
 *      caller enqueues on nn_stream) are captured instead of run; nn_plan_launch replays them
 *      in order on the stream, with the same results as the calls made one by one.
 *      Runs of consecutive single-token (M = 1) operators are replayed as ONE resident launch
 *      each: its blocks walk the run's operators, stream every operator's weights ahead of time
 *      and hand activations from operator to operator through device memory, so the replay
 *      pays no per-operator launch.  An operator joins a run when each buffer it reads is
 *      either untouched by the run so far or exactly one earlier operator's output (the whole
 *      buffer); other operators, M > 1 calls, row-sharded calls and the caller's own kernels
 *      stay separate launches between the runs.  A plan is replayed on its context's stream
 *      only, one replay at a time. ------------------------------------------------------- */
int nn_plan_begin(nn_context* ctx);
int nn_plan_end(nn_context* ctx, nn_plan** out_plan);
int nn_plan_launch(nn_context* ctx, nn_plan* plan);
int nn_plan_num_kernels(const nn_plan* plan);       /* launches per replay */
int nn_plan_num_recorded(const nn_plan* plan);      /* launches that were recorded */
int nn_plan_num_resident_runs(const nn_plan* plan); /* resident launches among them */
int nn_plan_free(nn_plan* plan);
/* Limit of every device-side wait inside the plan's resident launches (default about 200 ms,
 * 1..10000).  When a wait runs out the launch ends early, the next nn_sync returns
 * NN_ERR_TIMEOUT and the context stays usable.  No counterpart in the reference. */
int nn_plan_set_wait_limit(nn_plan* plan, unsigned timeout_ms);
/* Fault injection on the host side, for tests of that time-out: operator `op_index` of
 * resident run `run_index` computes but never hands its outputs to the operators that wait
 * for them (-1 restores normal behaviour).  No counterpart in the reference. */
int nn_plan_withhold_output(nn_plan* plan, int run_index, int op_index);
/* The grouping rule of nn_plan_end on address ranges alone (needs no GPU): operator i reads
 * x_addr[i] .. + x_bytes[i], writes its nout[i] <= 4 outputs out_addr[4*i + k] .. + out_bytes[4*i + k];
 * flags[i] bit 0: in-place epilogue (reads output 0 before writing it), bit 1: the last output is
 * the 4-byte index of a fused greedy pick.  Returns how many operators from `first` on may share a
 * resident launch and, for each of them, the operator (relative to `first`, -1 = not in the run)
 * that produces its x and its in-place values, a bit mask of outputs it still stores to memory
 * (an output overwritten later in the run is not stored) and of outputs it hands to later
 * operators.  No counterpart in the reference. */
int nn_plan_analyze(int nops, const uint64_t* x_addr, const uint64_t* x_bytes, const uint64_t* out_addr, const uint64_t* out_bytes,
                    const int* nout, const int* flags, int first, int* x_dep, int* res_dep, int* store_mask, int* publish_mask);

/* ---- class Weights, src/models/lfm2-5-350m/src/weights.h:13-51 (weights.cpp:169-297):
 *      mmap model.{fp16,int8,q4}.bin, parse meta.json, upload a tensor on first use. - */
int nn_weights_load(nn_context* ctx, const char* bin_path, const char* meta_path, nn_weights** out);
int nn_weights_free(nn_weights* w);
int nn_weights_has_tensor(const nn_weights* w, const char* key);
nn_buf nn_weights_get_buffer(nn_weights* w, const char* key, int optional); /* NULL when missing */
const char* nn_weights_get_dtype(const nn_weights* w, const char* key);     /* "" when missing */
int nn_weights_get_shape(const nn_weights* w, const char* key, int* dims, int max_dims); /* returns rank */
size_t nn_weights_get_size_bytes(const nn_weights* w, const char* key);
size_t nn_weights_get_num_elements(const nn_weights* w, const char* key);
int nn_weights_num_keys(const nn_weights* w);
const char* nn_weights_key_at(const nn_weights* w, int index); /* all_keys(), sorted */
int nn_weights_get_host_f32(const nn_weights* w, const char* key, float* out, size_t max_elems); /* get_host_vec */
/* The NNOPT_QUANT registration walk of src/models/lfm2-5-350m/src/main.cpp:527-566:
 * registers every int8 / q4_packed tensor that has a ".scale" sibling.
 * Returns the number registered (>= 0) or a negative code. */
int nn_weights_register_quantized(nn_context* ctx, nn_weights* w);

/* ---- timing: the per-launch OpenCL-event profilers
 *      (src/models/lfm2-5-350m/src/kernel_profiler.cpp:18-62) become CUDA events
 *      on the context's stream. --------------------------------------------------- */
int nn_event_create(void** out_event);
int nn_event_record(nn_context* ctx, void* event);
int nn_event_elapsed_ms(void* start, void* stop, float* out_ms); /* waits for stop */
int nn_event_destroy(void* event);
/* NNOPT_KERNEL_PROFILE=1 (or NNOPT_PROFILE=1) in the environment at nn_init switches the per-launch
 * profile on, the reference's switches of the same names (src/models/lfm2-5-350m/src/
 * kernel_profiler.cpp:18-62, src/models/smollm2-135m-instruct/src/prof.cpp:36-131): every call is
 * bracketed by a CUDA event pair under a label of the reference's form (gemv_m1_K1024_N4608_int8, with
 * the fused form appended; a plan replay is one entry), and nn_shutdown prints the table (label,
 * total ms, share, calls, average and maximum us; largest first) to stderr, as the reference does at
 * exit.  nn_profile_report formats the table so far into buf (returns its length; reset != 0 clears
 * the sums).  nn_profile_aggregate is the same aggregation and table on given (label, us) samples: it
 * needs no GPU. */
int nn_profile_enabled(const nn_context* ctx);
int nn_profile_report(nn_context* ctx, char* buf, size_t cap, int reset);
int nn_profile_aggregate(int n, const char* const* labels, const double* us, char* buf, size_t cap);
/* Read-bandwidth probe, the library's own measured ceiling for its weight streams: run_bw_probe,
 * src/models/lfm2-5-350m/src/main.cpp:29-139 with gemv_stream_buf / gemv_stream_img
 * (kernels/gemv_m1.cl:537-589).  Reads `bytes` (0: the larger of 1 GiB and eight times L2) of a
 * scratch buffer it allocates and frees, once untimed and once timed per trial, and reports the best
 * trial in GB/s (1e9 bytes) for the two read paths of this GPU: 16-byte loads by every thread, and
 * bulk copies into shared memory by the TMA unit, the path the streaming kernels use (where the
 * reference has buffer and image reads).  Either output may be NULL.  Synchronises the stream. */
int nn_bandwidth_probe(nn_context* ctx, size_t bytes, int trials, double* out_loads_gbs, double* out_tma_gbs);
/* Evict L2 between timed runs by rewriting a library-owned buffer larger than L2. */
int nn_l2_flush(nn_context* ctx);
/* Kernels launched by this context so far (for launch accounting). */
long long nn_launch_count(const nn_context* ctx);

/* ---- row sharding across GPUs (no counterpart in the reference, which is
 *      single-device; it extends the reference's own row tiling of large weights,
 *      src/models/lfm2-5-350m/src/utils.cpp:427-452, from image tiles to ranks).
 *      Rank g owns rows [g*N/G, (g+1)*N/G) of W and its scales; x is replicated;
 *      nn_comm_all_gather concatenates the per-rank [M, N/G] blocks in rank order:
 *      gathered layout is [G][M][N/G].  NCCL is loaded at run time (dlopen). ------ */
int nn_comm_unique_id(void* out_id_128bytes);
int nn_comm_init(nn_context* ctx, const void* id_128bytes, int rank, int world, nn_comm** out);
int nn_comm_all_gather(nn_comm* comm, nn_buf send, nn_buf recv, size_t bytes_per_rank);
int nn_comm_free(nn_comm* comm);

/* Projection fused with its gather, over peer-mapped memory (NVLink / NVSwitch):
 *   nn_comm_symm_alloc  collective; every rank passes the same size and gets a zeroed local
 *                       buffer whose twins on the other ranks are mapped here (CUDA IPC; needs
 *                       peer access between the GPUs, at most 8 ranks).  Freed with
 *                       nn_comm_symm_free (collective, after all ranks have synchronised) or
 *                       by nn_comm_free.
 *   nn_linear_gather    out block = x[M,K] . W[n_local,K]^T like nn_linear, where W holds this
 *                       rank's rows.  The kernel stores each output into block `rank` of the
 *                       gather buffer ([G][M][n_local] fp16) on EVERY rank, then the ranks
 *                       exchange completion flags; when the call's work has run in stream
 *                       order, all G blocks of this rank's `gathered` are complete.  `gathered`
 *                       must be a pointer returned by nn_comm_symm_alloc.  A peer may start
 *                       writing the next call's block into the same buffer while this rank
 *                       still reads it: alternate between two gather buffers.
 *   nn_comm_signal      publish "my stream has reached this point" to every rank;
 *   nn_comm_wait        hold the stream until every rank's signal count has reached this
 *                       rank's wait count, at most timeout_ms (1..10000); when the wait runs
 *                       out the next nn_sync returns NN_ERR_TIMEOUT and the context stays usable.
 *   nn_linear_argmax_sharded  greedy pick over a row-sharded lm_head (M = 1) without moving the
 *                       logits: rank g holds rows [g*n_local, (g+1)*n_local) of the weight; each
 *                       rank's projection kernel folds its rows into one (value, row) key and
 *                       stores it, tagged with the pick's number, in a table on every rank (one
 *                       8-byte peer store per rank, no fence: the word is its own arrival mark);
 *                       a one-warp kernel then waits (bounded, 2 s) for the G words and takes the
 *                       best.  Every rank's out_index (device int) receives the index
 *                       nn_linear_argmax would give on the whole weight (lowest row on ties, -1
 *                       when all values are NaN).  8 bytes per rank cross NVLink instead of 2*N.
 *                       `logits_local_fp16` may be NULL; otherwise this rank's n_local logits are
 *                       also stored there (ordinary device memory).  Every rank must make the
 *                       same sequence of these calls.  Needs one prior nn_comm_symm_alloc on the
 *                       communicator (which creates the flag and key words).
 *   nn_linear_argmax_sharded_rows  the same pick for M activation rows at once (batched greedy decode,
 *                       1 <= M <= 1024): each rank projects its rows of the weight into
 *                       logits_local ([M][n_local] fp16, ordinary device memory, required), folds every
 *                       row's n_local values into one key and stores the M keys in a table on every
 *                       rank; out_index receives M device ints.  8*M bytes per rank cross NVLink
 *                       instead of 2*M*N.  The first call allocates the key tables (collective; make
 *                       it outside a recording).
 *   nn_comm_pick_unsent fault injection on the host: one pick round, counted like any other, in
 *                       which no rank stores its key.  The waiting kernel must give up after
 *                       timeout_ms (1..10000), write -1 to out_index, and the next nn_sync must
 *                       return NN_ERR_TIMEOUT with the context and the communicator usable.
 *                       Every rank makes the call (or none).
 * No counterpart in the reference. */
int nn_comm_symm_alloc(nn_comm* comm, size_t bytes, nn_buf* out);
int nn_comm_symm_free(nn_comm* comm, nn_buf buf);
int nn_linear_gather(nn_comm* comm, int M, int n_local, int K, nn_buf x, nn_buf W, nn_buf gathered);
int nn_linear_argmax_sharded(nn_comm* comm, int n_local, int K, nn_buf x, nn_buf W, nn_buf logits_local_fp16, nn_buf out_index_i32);
int nn_linear_argmax_sharded_rows(nn_comm* comm, int M, int n_local, int K, nn_buf x, nn_buf W, nn_buf logits_local_fp16, nn_buf out_index_i32);
int nn_comm_pick_unsent(nn_comm* comm, unsigned timeout_ms, nn_buf out_index_i32);
int nn_comm_signal(nn_comm* comm);
int nn_comm_wait(nn_comm* comm, unsigned timeout_ms);
/* Number of CUDA devices visible to the process (0 when there is none). */
int nn_device_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NNOPT_B200_H */
