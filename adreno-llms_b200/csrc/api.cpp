// C-ABI layer: context, buffers, quantised-weight registry, operator dispatch,
// recorded decode steps, timing.  Declarations and the reference interfaces they
// replace are in include/nnopt_b200.h.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/nnopt_b200.h"
#include "internal.h"
#include "kernels.h"
#include "plan.h"

using namespace nnb;

// ---------------------------------------------------------------------------------
// errors: same shape as the reference's NNOPT_ERROR_FMT (always on, prints where)
// ---------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

int nnb::fail(int code, const char* file, int line, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    const char* base = strrchr(file, '/');
    fprintf(stderr, "ERROR: %s (%s:%d)\n", g_err, base ? base + 1 : file, line);
    return code;
}

extern "C" const char* nn_last_error(void) { return g_err; }
extern "C" const char* nn_version(void) { return "nnopt_b200 0.1 (sm_100a)"; }

#define CUDA_TRY(call)                                                                        \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

// ---------------------------------------------------------------------------------
// per-launch profile (NNOPT_KERNEL_PROFILE=1 or NNOPT_PROFILE=1)
// ---------------------------------------------------------------------------------
namespace {

const char* fmt_name(int fmt) { return fmt == FMT_FP16 ? "fp16" : fmt == FMT_INT8 ? "int8" : "q4"; }

// Labels in the reference's form, e.g. gemv_m1_K1024_N4608_int8 (utils.cpp:519 of the lfm2 port),
// with the fused form appended.
std::string op_label(int M, int N, int K, int fmt, const char* form) {
    char b[96];
    if (M == 1) snprintf(b, sizeof(b), "gemv_m1_K%d_N%d_%s%s", K, N, fmt_name(fmt), form);
    else snprintf(b, sizeof(b), "gemm_M%d_K%d_N%d_%s%s", M, K, N, fmt_name(fmt), form);
    return b;
}

struct ProfScope {  // event pair around whatever the scope enqueues
    nn_context* c;
    size_t slot = (size_t)-1;
    ProfScope(nn_context* ctx, const std::string& label) : c(ctx) {
        if (!c || !c->profiling || c->capturing) return;
        ProfPending p;
        p.label = label;
        if (cudaEventCreate(&p.start) != cudaSuccess) return;
        if (cudaEventCreate(&p.stop) != cudaSuccess) { cudaEventDestroy(p.start); return; }
        cudaEventRecord(p.start, c->stream);
        c->prof_pending.push_back(p);
        slot = c->prof_pending.size() - 1;
    }
    ~ProfScope() {
        if (slot != (size_t)-1) cudaEventRecord(c->prof_pending[slot].stop, c->stream);
    }
};

void prof_add(std::map<std::string, ProfAgg>& agg, const std::string& label, double us) {
    ProfAgg& a = agg[label];
    a.count++;
    a.total_us += us;
    if (us > a.max_us) a.max_us = us;
}

void prof_collect(nn_context* c) {
    if (c->prof_pending.empty()) return;
    cudaStreamSynchronize(c->stream);
    for (ProfPending& p : c->prof_pending) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, p.start, p.stop) == cudaSuccess) prof_add(c->prof, p.label, (double)ms * 1e3);
        cudaEventDestroy(p.start);
        cudaEventDestroy(p.stop);
    }
    c->prof_pending.clear();
}

// The table of the reference's dump, largest total first.
std::string prof_format(const std::map<std::string, ProfAgg>& agg) {
    std::vector<std::pair<std::string, ProfAgg>> rows(agg.begin(), agg.end());
    std::sort(rows.begin(), rows.end(), [](const std::pair<std::string, ProfAgg>& a, const std::pair<std::string, ProfAgg>& b) {
        return a.second.total_us != b.second.total_us ? a.second.total_us > b.second.total_us : a.first < b.first;
    });
    double grand = 0;
    for (const auto& r : rows) grand += r.second.total_us;
    char line[256];
    std::string out = "=== KERNEL PROFILE (env NNOPT_KERNEL_PROFILE=1) ===\n";
    snprintf(line, sizeof(line), "%-40s %12s %8s %12s %8s %8s\n", "label", "total_ms", "%total", "calls", "avg_us", "max_us");
    out += line;
    for (const auto& r : rows) {
        const ProfAgg& a = r.second;
        snprintf(line, sizeof(line), "%-40s %12.3f %7.2f%% %12llu %8.2f %8.2f\n", r.first.c_str(), a.total_us / 1e3,
                 grand > 0 ? 100.0 * a.total_us / grand : 0.0, a.count, a.count ? a.total_us / (double)a.count : 0.0, a.max_us);
        out += line;
    }
    snprintf(line, sizeof(line), "=== TOTAL GPU kernel time: %.3f ms ===\n", grand / 1e3);
    out += line;
    return out;
}

}  // namespace

extern "C" int nn_profile_enabled(const nn_context* c) { return c && c->profiling ? 1 : 0; }

extern "C" int nn_profile_report(nn_context* c, char* buf, size_t cap, int reset) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "nn_profile_report: null context");
    prof_collect(c);
    const std::string s = prof_format(c->prof);
    if (buf && cap) {
        const size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    if (reset) c->prof.clear();
    return (int)s.size();
}

extern "C" int nn_profile_aggregate(int n, const char* const* labels, const double* us, char* buf, size_t cap) {
    if (n < 0 || (n && (!labels || !us))) return NN_FAIL(NN_ERR_ARG, "nn_profile_aggregate: bad argument");
    std::map<std::string, ProfAgg> agg;
    for (int i = 0; i < n; ++i) prof_add(agg, labels[i] ? labels[i] : "", us[i]);
    const std::string s = prof_format(agg);
    if (buf && cap) {
        const size_t m = s.size() < cap - 1 ? s.size() : cap - 1;
        memcpy(buf, s.data(), m);
        buf[m] = 0;
    }
    return (int)s.size();
}

// ---------------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------------
extern "C" int nn_init(int device, nn_context** out) {
    if (!out) return NN_FAIL(NN_ERR_ARG, "nn_init: out_ctx is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return NN_FAIL(NN_ERR_CUDA, "nn_init: no CUDA device (%s); this library has no CPU path",
                       e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    if (device < 0 || device >= count) return NN_FAIL(NN_ERR_ARG, "nn_init: device %d out of range [0,%d)", device, count);
    CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return NN_FAIL(NN_ERR_UNSUPPORTED, "nn_init: device %d is sm_%d%d; the kernels are built for sm_100a only", device,
                       prop.major, prop.minor);
    nn_context* c = new nn_context();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->l2_bytes = (size_t)prop.l2CacheSize;
    c->hbm_bytes = prop.totalGlobalMem;
    c->smem_limit = prop.sharedMemPerBlockOptin;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete c;
        return NN_FAIL(NN_ERR_CUDA, "nn_init: cudaStreamCreate failed");
    }
    if (cudaHostAlloc((void**)&c->status_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void**)&c->status_dev, c->status_host, 0) != cudaSuccess) {
        delete c;
        return NN_FAIL(NN_ERR_CUDA, "nn_init: status word allocation failed");
    }
    *c->status_host = 0;
    // [0] nn_argmax's reduction word, [1] the fused arg-max's word, [2] its block counter
    if (cudaMalloc((void**)&c->argmax_slot, 32) != cudaSuccess || cudaMemset(c->argmax_slot, 0, 32) != cudaSuccess) {
        delete c;
        return NN_FAIL(NN_ERR_CUDA, "nn_init: cudaMalloc failed");
    }
    if (cudaMalloc((void**)&c->sk_scratch, SK_SCRATCH_BYTES) != cudaSuccess ||
        cudaMalloc((void**)&c->sk_flags, SK_MAX_BLOCKS * sizeof(unsigned)) != cudaSuccess ||
        cudaMemset(c->sk_flags, 0, SK_MAX_BLOCKS * sizeof(unsigned)) != cudaSuccess) {
        delete c;
        return NN_FAIL(NN_ERR_CUDA, "nn_init: cudaMalloc failed");
    }
    // normalised activations for the norm-then-project calls that cannot fuse the norm: sized for the
    // decode shapes up front so that such calls also work inside a recording (it grows outside one)
    // the staged activations of a batched call never exceed the shared memory of one block
    c->stage_img_bytes = (size_t)256 << 10;
    if (cudaMalloc(&c->stage_img, c->stage_img_bytes) != cudaSuccess || cudaMemset(c->stage_img, 0, c->stage_img_bytes) != cudaSuccess) {
        delete c;
        return NN_FAIL(NN_ERR_CUDA, "nn_init: cudaMalloc failed");
    }
    c->norm_scratch_bytes = (size_t)1 << 20;
    if (cudaMalloc(&c->norm_scratch, c->norm_scratch_bytes) != cudaSuccess) {
        delete c;
        return NN_FAIL(NN_ERR_CUDA, "nn_init: cudaMalloc failed");
    }
    if ((e = stream_configure()) != cudaSuccess) {
        delete c;
        return NN_FAIL(NN_ERR_CUDA, "nn_init: kernel configuration failed: %s", cudaGetErrorString(e));
    }
    const char* pdl = getenv("NNB_PDL");
    c->use_pdl = !(pdl && pdl[0] == '0');
    const char* kp = getenv("NNOPT_KERNEL_PROFILE");
    const char* pp = getenv("NNOPT_PROFILE");
    c->profiling = (kp && kp[0] == '1') || (pp && pp[0] == '1');
    *out = c;
    return NN_OK;
}

extern "C" int nn_shutdown(nn_context* c) {
    if (!c) return NN_OK;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    if (c->profiling) {  // the reference dumps its per-kernel table when the program ends
        prof_collect(c);
        if (!c->prof.empty()) fprintf(stderr, "\n%s\n", prof_format(c->prof).c_str());
    }
    for (auto& kv : c->registry) free_scale_pad(kv.second);
    if (c->flush_buf) cudaFree(c->flush_buf);
    if (c->argmax_slot) cudaFree(c->argmax_slot);
    if (c->norm_scratch) cudaFree(c->norm_scratch);
    if (c->stage_img) cudaFree(c->stage_img);
    if (c->pair_scratch) cudaFree(c->pair_scratch);
    if (c->sk_scratch) cudaFree(c->sk_scratch);
    if (c->sk_flags) cudaFree(c->sk_flags);
    if (c->status_host) cudaFreeHost(c->status_host);
    cudaStreamDestroy(c->stream);
    delete c;
    return NN_OK;
}

extern "C" int nn_device_count(void) {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess ? n : 0;
}

extern "C" void* nn_stream(nn_context* c) { return c ? (void*)c->stream : nullptr; }

extern "C" int nn_sync(nn_context* c) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "nn_sync: null context");
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    if (*c->status_host != 0) {
        const int s = *c->status_host;
        *c->status_host = 0;
        cudaMemsetAsync(c->argmax_slot, 0, 32, c->stream);  // a cut-short launch may have left its words set
        cudaMemsetAsync(c->sk_flags, 0, SK_MAX_BLOCKS * sizeof(unsigned), c->stream);
        return NN_FAIL(NN_ERR_TIMEOUT, "a device-side bounded wait ran out (status %d); results of the last calls are invalid", s);
    }
    return NN_OK;
}

extern "C" int nn_device_info(nn_context* c, int* sm, size_t* l2, size_t* hbm) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "nn_device_info: null context");
    if (sm) *sm = c->sm_count;
    if (l2) *l2 = c->l2_bytes;
    if (hbm) *hbm = c->hbm_bytes;
    return NN_OK;
}

extern "C" long long nn_launch_count(const nn_context* c) { return c ? c->launches : 0; }

// ---------------------------------------------------------------------------------
// buffers
// ---------------------------------------------------------------------------------
extern "C" nn_buf nn_buf_alloc(nn_context* c, size_t bytes) {
    if (!c) { NN_FAIL(NN_ERR_ARG, "nn_buf_alloc: null context"); return nullptr; }
    cudaSetDevice(c->device);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess) { NN_FAIL(NN_ERR_CUDA, "nn_buf_alloc(%zu): %s", bytes, cudaGetErrorString(e)); return nullptr; }
    return p;
}
extern "C" int nn_buf_free(nn_context* c, nn_buf b) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "nn_buf_free: null context");
    if (!b) return NN_OK;
    cudaSetDevice(c->device);
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    // a freed weight or scale buffer must not keep resolving: the address may be handed out again
    for (auto it = c->registry.begin(); it != c->registry.end();) {
        if (it->first == (uintptr_t)b || (const void*)it->second.scale == (const void*)b) {
            free_scale_pad(it->second);
            it = c->registry.erase(it);
        }
        else ++it;
    }
    CUDA_TRY(cudaFree(b));
    return NN_OK;
}
extern "C" int nn_buf_write(nn_context* c, nn_buf dst, size_t off, const void* src, size_t bytes) {
    if (!c || !dst || (!src && bytes)) return NN_FAIL(NN_ERR_ARG, "nn_buf_write: null argument");
    if (!bytes) return NN_OK;
    CUDA_TRY(cudaMemcpyAsync((char*)dst + off, src, bytes, cudaMemcpyHostToDevice, c->stream));
    return NN_OK;
}
extern "C" int nn_buf_read(nn_context* c, void* dst, nn_buf src, size_t off, size_t bytes) {
    if (!c || !src || (!dst && bytes)) return NN_FAIL(NN_ERR_ARG, "nn_buf_read: null argument");
    if (!bytes) return NN_OK;
    CUDA_TRY(cudaMemcpyAsync(dst, (const char*)src + off, bytes, cudaMemcpyDeviceToHost, c->stream));
    return NN_OK;
}
extern "C" int nn_buf_copy(nn_context* c, nn_buf dst, nn_buf src, size_t bytes) {
    if (!c || !dst || !src) return NN_FAIL(NN_ERR_ARG, "nn_buf_copy: null argument");
    if (!bytes) return NN_OK;
    CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, c->stream));
    return NN_OK;
}
extern "C" int nn_buf_fill(nn_context* c, nn_buf dst, int v, size_t bytes) {
    if (!c || !dst) return NN_FAIL(NN_ERR_ARG, "nn_buf_fill: null argument");
    if (!bytes) return NN_OK;
    CUDA_TRY(cudaMemsetAsync(dst, v, bytes, c->stream));
    return NN_OK;
}
extern "C" void* nn_host_alloc(size_t bytes) {
    void* p = nullptr;
    cudaError_t e = cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault);
    if (e != cudaSuccess) { NN_FAIL(NN_ERR_CUDA, "nn_host_alloc(%zu): %s", bytes, cudaGetErrorString(e)); return nullptr; }
    return p;
}
extern "C" int nn_host_free(void* p) {
    if (p) CUDA_TRY(cudaFreeHost(p));
    return NN_OK;
}

// ---------------------------------------------------------------------------------
// registry
// ---------------------------------------------------------------------------------
static size_t fmt_rowbytes(int fmt, int K) { return fmt == FMT_FP16 ? (size_t)K * 2 : fmt == FMT_INT8 ? (size_t)K : (size_t)K / 2; }

static int register_weight(nn_context* c, int fmt, nn_buf W, nn_buf scale, int N, int K, const char* who) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "%s: null context", who);
    if (!W || !scale) return NN_FAIL(NN_ERR_ARG, "%s: null weight or scale buffer", who);
    if (N <= 0 || K <= 0) return NN_FAIL(NN_ERR_ARG, "%s: bad shape N=%d K=%d", who, N, K);
    if (fmt == FMT_Q4 && (K % 32) != 0) return NN_FAIL(NN_ERR_ARG, "%s: Q4 needs K %% 32 == 0, got K=%d", who, K);
    QuantEntry q;
    q.fmt = fmt;
    q.scale = (const uint16_t*)scale;
    q.N = N;
    q.K = K;
    q.rowbytes = fmt_rowbytes(fmt, K);
    auto old = c->registry.find((uintptr_t)W);
    if (old != c->registry.end()) free_scale_pad(old->second);
    if (fmt == FMT_Q4 && (K / 16) % 16 != 0 && !c->capturing) {
        // scale rows of K / 16 bytes that tensor copies cannot address: keep a copy with 16-byte row pitch
        const size_t src_pitch = (size_t)K / 16, pitch = (src_pitch + 15) / 16 * 16;
        cudaSetDevice(c->device);
        void* pad = nullptr;
        if (cudaMalloc(&pad, pitch * (size_t)N) == cudaSuccess) {
            if (cudaMemsetAsync(pad, 0, pitch * (size_t)N, c->stream) == cudaSuccess &&
                cudaMemcpy2DAsync(pad, pitch, scale, src_pitch, src_pitch, (size_t)N, cudaMemcpyDeviceToDevice, c->stream) == cudaSuccess) {
                q.scale_pad = (uint16_t*)pad;
                q.scale_pitch = (int)pitch;
            } else {
                cudaFree(pad);
                cudaGetLastError();
            }
        } else {
            cudaGetLastError();   // no memory for the copy: the per-lane scale path still works
        }
    }
    c->registry[(uintptr_t)W] = q;
    return NN_OK;
}

extern "C" int nn_register_int8_weight(nn_context* c, nn_buf W, nn_buf s, int N, int K) {
    return register_weight(c, FMT_INT8, W, s, N, K, "nn_register_int8_weight");
}
extern "C" int nn_register_q4_weight(nn_context* c, nn_buf W, nn_buf s, int N, int K) {
    return register_weight(c, FMT_Q4, W, s, N, K, "nn_register_q4_weight");
}
extern "C" int nn_unregister_weight(nn_context* c, nn_buf W) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "nn_unregister_weight: null context");
    auto it = c->registry.find((uintptr_t)W);
    if (it != c->registry.end()) {
        free_scale_pad(it->second);
        c->registry.erase(it);
    }
    return NN_OK;
}

// Resolve W to (format, scale pointer for its first row, rows available).  A pointer
// inside a registered weight at a whole-row offset is a row-range view of it.
bool nnb::resolve_weight(const nn_context* c, const void* W, int K, ResolvedW* out) {
    out->fmt = FMT_FP16;
    out->scale = nullptr;
    out->rows_avail = -1;
    out->scale_pad = nullptr;
    out->scale_pitch = 0;
    if (c->registry.empty()) return true;
    const uintptr_t p = (uintptr_t)W;
    auto it = c->registry.upper_bound(p);
    if (it == c->registry.begin()) return true;
    --it;
    const QuantEntry& q = it->second;
    const uintptr_t base = it->first;
    const size_t span = q.rowbytes * (size_t)q.N;
    if (p >= base + span) return true;  // not inside any registered weight: fp16
    const size_t off = p - base;
    if (off % q.rowbytes) return false;  // inside a quantised weight but not on a row boundary
    if (q.K != K) return false;
    const size_t r = off / q.rowbytes;
    out->fmt = q.fmt;
    out->scale = q.fmt == FMT_INT8 ? q.scale + r : q.scale + r * (size_t)(K / 32);
    out->rows_avail = q.N - (int)r;
    if (q.scale_pad) {
        out->scale_pad = reinterpret_cast<const uint16_t*>(reinterpret_cast<const char*>(q.scale_pad) + r * (size_t)q.scale_pitch);
        out->scale_pitch = q.scale_pitch;
    }
    return true;
}

// ---------------------------------------------------------------------------------
// operator dispatch
// ---------------------------------------------------------------------------------
// M > 16 with one weight and a plain or residual epilogue: tensor-core GEMM (quantised weights
// are expanded to fp16 inside the kernel, stage by stage).
static int run_gemm_tc(nn_context* c, int fmt, const LinArgs& a, int M, const char* who, bool* done) {
    *done = false;
    if (a.nseg != 1 || !(a.epi == EPI_STORE || a.epi == EPI_RESIDUAL)) return NN_OK;
    const LinSeg& sg = a.seg[0];
    if (!gemm_tc_supported(fmt, M, sg.N, a.K, a.x, sg.W, sg.out)) return NN_OK;
    cudaError_t e = launch_gemm_tc(fmt, sg.W, sg.scale, a.x, sg.out, M, sg.N, a.K, sg.ld_out, a.epi, a.status, a.peer_out, a.npeer, &a.sig, c->stream);
    if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "%s: tensor-core launch failed: %s (M=%d N=%d K=%d)", who, cudaGetErrorString(e), M, sg.N, a.K);
    c->launches++;
    *done = true;
    return NN_OK;
}

// The fused forms (three-weight QKV, SwiGLU over two weights, the in-place SiLU gate) at prefill row counts: one
// tensor-core GEMM per weight, each with an fp16 result, and for the two-weight forms the element-wise SiLU-multiply
// over those results -- the reference's own M > 1 sequence (src/models/lfm2-5-350m/src/layers/mlp.cpp:101-129).  The
// single-pass streaming kernel would walk such a batch in slices of 16 rows, re-reading the weights for every slice.
static int run_fused_forms_tc(nn_context* c, int fmt, const LinArgs& a, int M, const char* who, bool* done) {
    *done = false;
    if (a.npeer > 0 || a.sig.world > 0 || a.argmax_slot || a.norm_w) return NN_OK;
    const bool qkv = a.epi == EPI_STORE && a.nseg > 1, swiglu = a.epi == EPI_SWIGLU && a.nseg == 1, gate = a.epi == EPI_SILU_GATE && a.nseg == 1;
    if (!qkv && !swiglu && !gate) return NN_OK;
    for (int i = 0; i < a.nseg; ++i)
        if (!gemm_tc_supported(fmt, M, a.seg[i].N, a.K, a.x, a.seg[i].W, a.seg[i].out)) return NN_OK;
    if (swiglu && !gemm_tc_supported(fmt, M, a.seg[0].N, a.K, a.x, a.W2, a.seg[0].out)) return NN_OK;
    auto gemm = [&](const uint8_t* W, const uint16_t* scale, uint16_t* out, int N, int ld) -> int {
        cudaError_t e = launch_gemm_tc(fmt, W, scale, a.x, out, M, N, a.K, ld, EPI_STORE, a.status, nullptr, 0, nullptr, c->stream);
        if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "%s: tensor-core launch failed: %s (M=%d N=%d K=%d)", who, cudaGetErrorString(e), M, N, a.K);
        c->launches++;
        return NN_OK;
    };
    if (qkv) {
        for (int i = 0; i < a.nseg; ++i) {
            const int rc = gemm(a.seg[i].W, a.seg[i].scale, a.seg[i].out, a.seg[i].N, a.seg[i].ld_out);
            if (rc) return rc;
        }
        *done = true;
        return NN_OK;
    }
    const int N = a.seg[0].N;
    const size_t one = (size_t)M * N * 2, need = swiglu ? 2 * one : one;
    if (need > c->pair_scratch_bytes) {
        if (c->capturing) return NN_OK;   // cannot grow inside a recording: the sliced route still works
        cudaSetDevice(c->device);
        CUDA_TRY(cudaStreamSynchronize(c->stream));
        if (c->pair_scratch) CUDA_TRY(cudaFree(c->pair_scratch));
        c->pair_scratch = nullptr;
        c->pair_scratch_bytes = 0;
        CUDA_TRY(cudaMalloc(&c->pair_scratch, need));
        c->pair_scratch_bytes = need;
    }
    uint16_t* s0 = (uint16_t*)c->pair_scratch;
    uint16_t* s1 = (uint16_t*)((char*)c->pair_scratch + one);
    if (swiglu) {
        int rc = gemm(a.seg[0].W, a.seg[0].scale, s0, N, N);
        if (!rc) rc = gemm(a.W2, a.scale2, s1, N, N);
        if (rc) return rc;
        CUDA_TRY(launch_silu_mul(s0, s1, a.seg[0].out, (size_t)M * N, c->stream));
    } else {   // gate_inout = silu(gate_inout) * (x . W3^T)
        const int rc = gemm(a.seg[0].W, a.seg[0].scale, s0, N, N);
        if (rc) return rc;
        if (a.seg[0].ld_out != N) return NN_FAIL(NN_ERR_UNSUPPORTED, "%s: the in-place gate form needs a dense [M, N] buffer", who);
        CUDA_TRY(launch_silu_mul(a.seg[0].out, s0, a.seg[0].out, (size_t)M * N, c->stream));
    }
    c->launches++;
    *done = true;
    return NN_OK;
}

// While a step is being recorded, every launch of the streaming kernel is also noted with its
// arguments and its graph node, so that nn_plan_end can hand runs of them to the resident kernel.
static void note_recorded(nn_context* c, int fmt, const LinArgs& a, const StreamPlan& p) {
    if (!c->capturing) return;
    RecordedOp r;
    r.fmt = fmt;
    r.a = a;
    r.p = p;
    r.node = nullptr;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    const cudaGraphNode_t* tail = nullptr;
    size_t ntail = 0;
    if (cudaStreamGetCaptureInfo(c->stream, &st, nullptr, nullptr, &tail, &ntail) == cudaSuccess && st == cudaStreamCaptureStatusActive && ntail == 1)
        r.node = tail[0];
    bool q4_ok = true;
    if (fmt == FMT_Q4) {  // block scales must be reachable by tensor copies
        const uint16_t* base[4];
        int pitch = 0;
        q4_ok = q4_scale_views(a, base, &pitch);
    }
    r.eligible = r.node && a.M == 1 && !p.streamk && a.npeer == 0 && a.sig.world == 0 && q4_ok;
    c->rec.push_back(r);
}

static int run_linear(nn_context* c, int fmt, LinArgs a, int M_total, const char* who) {
    a.sk_scratch = c->sk_scratch;
    a.sk_flags = c->sk_flags;
    if (a.norm_w) {
        // the prologue is fused into the streaming kernel; every other route normalises into
        // context scratch first
        LinArgs probe = a;
        probe.M = M_total;
        // a batched call (2..16 rows) normalises in the launch that stages its activations, so the
        // projection itself needs no room for the normalised rows
        if (M_total >= 2) probe.norm_w = nullptr;
        bool fused = M_total <= 16 && stream_supported(fmt, M_total, a.K, probe) && (M_total == 1 || (size_t)a.K * 2 <= ((size_t)48 << 10));
        if (fused) fused = stream_plan(fmt, probe, c->sm_count, c->smem_limit).ok;
        if (!fused) {
            const size_t need = (size_t)M_total * a.K * 2;
            if (need > c->norm_scratch_bytes) {
                if (c->capturing) return NN_FAIL(NN_ERR_UNSUPPORTED, "%s: the norm scratch cannot grow while a plan is being recorded; run the call once before recording", who);
                cudaSetDevice(c->device);
                CUDA_TRY(cudaStreamSynchronize(c->stream));
                if (c->norm_scratch) CUDA_TRY(cudaFree(c->norm_scratch));
                c->norm_scratch = nullptr;
                c->norm_scratch_bytes = 0;
                CUDA_TRY(cudaMalloc(&c->norm_scratch, need));
                c->norm_scratch_bytes = need;
            }
            CUDA_TRY(launch_rmsnorm(a.x, a.norm_w, (uint16_t*)c->norm_scratch, M_total, a.K, a.norm_eps, c->stream));
            c->launches++;
            a.x = (const uint16_t*)c->norm_scratch;
            a.norm_w = nullptr;
        }
    }
    if (M_total > 16) {
        bool done = false;
        int rc = run_gemm_tc(c, fmt, a, M_total, who, &done);
        if (rc != NN_OK || done) return rc;
        rc = run_fused_forms_tc(c, fmt, a, M_total, who, &done);
        if (rc != NN_OK || done) return rc;
    }
    // M > 16 is walked in slices of 16 activation rows (each slice re-streams the weights).
    const uint16_t* x0 = a.x;
    uint16_t* out0[3] = {a.seg[0].out, a.seg[1].out, a.seg[2].out};
    uint16_t* peer0[7];
    for (int p = 0; p < 7; ++p) peer0[p] = a.peer_out[p];
    const GatherSignal sig0 = a.sig;
    // Slices of at most 16 rows; when the activations of a slice do not fit in shared memory next
    // to the weight ring (large K, int8 limb planes), the slice is halved until they do.
    int slice = 16;
    {
        LinArgs probe = a;
        if (M_total >= 2) probe.norm_w = nullptr;
        while (slice > 1) {
            probe.M = M_total < slice ? M_total : slice;
            if (!stream_supported(fmt, probe.M, a.K, probe) || stream_plan(fmt, probe, c->sm_count, c->smem_limit).ok) break;
            slice >>= 1;
        }
    }
    for (int m0 = 0; m0 < M_total; m0 += slice) {
        a.sig = sig0;
        if (m0 + slice < M_total) a.sig.world = 0;  // the last slice sends the gather's signal
        a.M = M_total - m0 < slice ? M_total - m0 : slice;
        a.x = x0 + (size_t)m0 * a.K;
        for (int i = 0; i < a.nseg; ++i) a.seg[i].out = out0[i] + (size_t)m0 * a.seg[i].ld_out;
        for (int p = 0; p < a.npeer; ++p) a.peer_out[p] = peer0[p] + (size_t)m0 * a.seg[0].ld_out;
        cudaError_t e;
        StreamPlan p = {};
        LinArgs b = a;
        // Measured on whole batched steps: int8 and fp16 always gain from the staging launch; Q4 rows are cheap to
        // stage in place, so it pays only from about 12K activation values (or when there is a norm to apply)
        const bool stage_pays = fmt != FMT_Q4 || (long long)a.M * a.K >= 12288 || a.norm_w != nullptr;
        if (a.M >= 2 && stage_pays && stream_supported(fmt, a.M, a.K, a) && stage_image_bytes(fmt, a.M, a.K) <= c->stage_img_bytes) {
            // batched: the activations (normalised when asked) are staged once, by a launch of their own
            b.norm_w = nullptr;
            b.staged = (const uint8_t*)c->stage_img;
            b.staged_bytes = (unsigned)stage_image_bytes(fmt, a.M, a.K);
            p = stream_plan(fmt, b, c->sm_count, c->smem_limit);
            if (p.ok) {
                e = launch_stage_image(fmt, a.x, a.M, a.K, a.norm_w, a.norm_eps, (uint8_t*)c->stage_img, c->stream, c->use_pdl);
                if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "%s: staging launch failed: %s (M=%d K=%d)", who, cudaGetErrorString(e), a.M, a.K);
                c->launches++;
            } else {
                b = a;
            }
        }
        if (!p.ok && stream_supported(fmt, a.M, a.K, a)) p = stream_plan(fmt, a, c->sm_count, c->smem_limit);
        if (p.ok) {
            e = launch_stream(fmt, b, p, c->stream, c->use_pdl);
            if (e == cudaSuccess && M_total == 1) note_recorded(c, fmt, a, p);
        } else {
            if (a.npeer > 0)
                return NN_FAIL(NN_ERR_UNSUPPORTED, "%s: this shape takes the any-shape kernel, which does not write to peer ranks (K=%d)", who, a.K);
            e = launch_generic(fmt, a, c->stream);
        }
        if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "%s: launch failed: %s (M=%d K=%d)", who, cudaGetErrorString(e), a.M, a.K);
        c->launches++;
    }
    return NN_OK;
}

static int check_common(nn_context* c, int M, int N, int K, const void* x, const void* W, const void* out, const char* who) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "%s: null context", who);
    if (!x || !W || !out) return NN_FAIL(NN_ERR_ARG, "%s: null buffer (x=%p W=%p out=%p)", who, x, W, out);
    if (M < 0 || N <= 0 || K <= 0) return NN_FAIL(NN_ERR_ARG, "%s: bad shape M=%d N=%d K=%d", who, M, N, K);
    return NN_OK;
}

// `gamma` (with `eps`): RMSNorm of the activations before the projection, or null.
static int one_weight(nn_context* c, int M, int N, int K, nn_buf x, nn_buf W, nn_buf out, int epi, const char* who,
                      uint16_t* const* peers = nullptr, int npeer = 0, const GatherSignal* sig = nullptr, nn_buf gamma = nullptr, float eps = 0.f) {
    int rc = check_common(c, M, N, K, x, W, out, who);
    if (rc) return rc;
    if (M == 0) return NN_OK;
    ResolvedW r;
    if (!resolve_weight(c, W, K, &r))
        return NN_FAIL(NN_ERR_ARG, "%s: W points into a registered quantised weight but K=%d or the row offset does not match", who, K);
    if (r.rows_avail >= 0 && N > r.rows_avail)
        return NN_FAIL(NN_ERR_ARG, "%s: N=%d exceeds the %d rows registered for this weight", who, N, r.rows_avail);
    LinArgs a = {};
    a.nseg = 1;
    a.seg[0].W = (const uint8_t*)W;
    a.seg[0].scale = r.scale;
    a.scale_pad[0] = r.scale_pad;
    a.scale_pitch = r.scale_pitch;
    a.seg[0].out = (uint16_t*)out;
    a.seg[0].N = N;
    a.seg[0].ld_out = N;
    a.x = (const uint16_t*)x;
    a.K = K;
    a.epi = epi;
    a.status = c->status_dev;
    a.norm_w = (const uint16_t*)gamma;
    a.norm_eps = eps;
    ProfScope prof(c, op_label(M, N, K, r.fmt, epi == EPI_RESIDUAL ? "_add" : epi == EPI_SILU_GATE ? "_silu_gate" : gamma ? "_rmsnorm" : ""));
    if (npeer < 0 || npeer > 7) return NN_FAIL(NN_ERR_ARG, "%s: %d peers", who, npeer);
    a.npeer = npeer;
    for (int p = 0; p < npeer; ++p) a.peer_out[p] = peers[p];
    if (sig) a.sig = *sig;
    return run_linear(c, r.fmt, a, M, who);
}

int nnb::linear_to_peers(nn_context* c, int M, int N, int K, nn_buf x, nn_buf W, nn_buf out, uint16_t* const* peers, int npeer,
                         const GatherSignal* sig, const char* who) {
    return one_weight(c, M, N, K, x, W, out, EPI_STORE, who, peers, npeer, sig);
}

extern "C" int nn_linear(nn_context* c, int M, int N, int K, nn_buf x, nn_buf W, nn_buf out) {
    return one_weight(c, M, N, K, x, W, out, EPI_STORE, "nn_linear");
}
extern "C" int nn_linear_add(nn_context* c, int M, int N, int K, nn_buf x, nn_buf W, nn_buf r) {
    return one_weight(c, M, N, K, x, W, r, EPI_RESIDUAL, "nn_linear_add");
}
extern "C" int nn_linear_silu_gate_fused(nn_context* c, int M, int N, int K, nn_buf x, nn_buf W3, nn_buf g) {
    return one_weight(c, M, N, K, x, W3, g, EPI_SILU_GATE, "nn_linear_silu_gate_fused");
}

static int gate_up_silu(nn_context* c, int M, int N, int K, nn_buf x, nn_buf Wg, nn_buf Wu, nn_buf out, nn_buf gamma, float eps, const char* who) {
    int rc = check_common(c, M, N, K, x, Wg, out, who);
    if (rc) return rc;
    if (!Wu) return NN_FAIL(NN_ERR_ARG, "%s: null Wu", who);
    if (M == 0) return NN_OK;
    ResolvedW rg, ru;
    if (!resolve_weight(c, Wg, K, &rg) || !resolve_weight(c, Wu, K, &ru))
        return NN_FAIL(NN_ERR_ARG, "%s: weight registration does not match K=%d", who, K);
    if (rg.fmt != ru.fmt) return NN_FAIL(NN_ERR_ARG, "%s: gate and up weights are of different formats", who);
    if ((rg.rows_avail >= 0 && N > rg.rows_avail) || (ru.rows_avail >= 0 && N > ru.rows_avail))
        return NN_FAIL(NN_ERR_ARG, "%s: N=%d exceeds the registered rows", who, N);
    LinArgs a = {};
    a.nseg = 1;
    a.seg[0].W = (const uint8_t*)Wg;
    a.seg[0].scale = rg.scale;
    a.scale_pad[0] = rg.scale_pad;
    a.scale_pad[3] = ru.scale_pad;
    a.scale_pitch = rg.scale_pitch;
    a.seg[0].out = (uint16_t*)out;
    a.seg[0].N = N;
    a.seg[0].ld_out = N;
    a.W2 = (const uint8_t*)Wu;
    a.scale2 = ru.scale;
    a.x = (const uint16_t*)x;
    a.K = K;
    a.epi = EPI_SWIGLU;
    a.status = c->status_dev;
    a.norm_w = (const uint16_t*)gamma;
    a.norm_eps = eps;
    ProfScope prof(c, op_label(M, N, K, rg.fmt, gamma ? "_rmsnorm_swiglu" : "_swiglu"));
    return run_linear(c, rg.fmt, a, M, who);
}

extern "C" int nn_fused_gate_up_silu(nn_context* c, int M, int N, int K, nn_buf x, nn_buf Wg, nn_buf Wu, nn_buf out) {
    return gate_up_silu(c, M, N, K, x, Wg, Wu, out, nullptr, 0.f, "nn_fused_gate_up_silu");
}

static int linear_qkv(nn_context* c, int M, int K, nn_buf x, nn_buf Wq, int Nq, nn_buf Wk, int Nk, nn_buf Wv, int Nv, nn_buf q, nn_buf k, nn_buf v,
                      nn_buf gamma, float eps, const char* who, nn_buf bq = nullptr, nn_buf bk = nullptr, nn_buf bv = nullptr) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "%s: null context", who);
    if (!x || !Wq || !Wk || !Wv || !q || !k || !v) return NN_FAIL(NN_ERR_ARG, "%s: null buffer", who);
    if (M < 0 || K <= 0 || Nq <= 0 || Nk <= 0 || Nv <= 0) return NN_FAIL(NN_ERR_ARG, "%s: bad shape", who);
    if (M == 0) return NN_OK;
    const void* Ws[3] = {Wq, Wk, Wv};
    void* outs[3] = {q, k, v};
    const int Ns[3] = {Nq, Nk, Nv};
    LinArgs a = {};
    a.nseg = 3;
    int fmt = -1;
    for (int i = 0; i < 3; ++i) {
        ResolvedW r;
        if (!resolve_weight(c, Ws[i], K, &r)) return NN_FAIL(NN_ERR_ARG, "%s: weight %d registration does not match K=%d", who, i, K);
        if (r.rows_avail >= 0 && Ns[i] > r.rows_avail) return NN_FAIL(NN_ERR_ARG, "%s: weight %d has fewer rows than asked", who, i);
        if (fmt >= 0 && r.fmt != fmt) return NN_FAIL(NN_ERR_ARG, "%s: the three weights are of different formats", who);
        fmt = r.fmt;
        a.seg[i].W = (const uint8_t*)Ws[i];
        a.seg[i].scale = r.scale;
        a.scale_pad[i] = r.scale_pad;
        a.scale_pitch = r.scale_pitch;
        a.seg[i].out = (uint16_t*)outs[i];
        a.seg[i].N = Ns[i];
        a.seg[i].ld_out = Ns[i];
    }
    a.x = (const uint16_t*)x;
    a.K = K;
    a.epi = EPI_STORE;
    a.status = c->status_dev;
    a.norm_w = (const uint16_t*)gamma;
    a.norm_eps = eps;
    if (bq) {
        // The bias rides in the projection's epilogue when the call takes the streaming kernel (up to 16 rows); otherwise
        // the projection runs as it would without one and the reference's bias kernel follows it.
        const void* bs[3] = {bq, bk, bv};
        bool fused = M <= 16;
        if (fused) {
            LinArgs probe = a;
            probe.M = M;
            if (M >= 2) probe.norm_w = nullptr;
            fused = stream_supported(fmt, M, K, probe) && stream_plan(fmt, probe, c->sm_count, c->smem_limit).ok;
        }
        if (fused) {
            for (int i = 0; i < 3; ++i) a.seg[i].bias = (const uint16_t*)bs[i];
            ProfScope prof(c, op_label(M, Nq + Nk + Nv, K, fmt, gamma ? "_rmsnorm_qkv_bias" : "_qkv_bias"));
            return run_linear(c, fmt, a, M, who);
        }
        int rc;
        {
            ProfScope prof(c, op_label(M, Nq + Nk + Nv, K, fmt, gamma ? "_rmsnorm_qkv" : "_qkv"));
            rc = run_linear(c, fmt, a, M, who);
        }
        if (rc) return rc;
        BiasArgs ba = {};
        for (int i = 0; i < 3; ++i) {
            ba.out[i] = (uint16_t*)outs[i];
            ba.bias[i] = (const uint16_t*)bs[i];
            ba.cols[i] = Ns[i];
        }
        ba.rows = M;
        ba.nseg = 3;
        ProfScope prof(c, "bias_add_qkv_rows" + std::to_string(M));
        CUDA_TRY(launch_bias_add(ba, c->stream));
        c->launches++;
        return NN_OK;
    }
    ProfScope prof(c, op_label(M, Nq + Nk + Nv, K, fmt, gamma ? "_rmsnorm_qkv" : "_qkv"));
    return run_linear(c, fmt, a, M, who);
}

extern "C" int nn_linear_qkv(nn_context* c, int M, int K, nn_buf x, nn_buf Wq, int Nq, nn_buf Wk, int Nk, nn_buf Wv, int Nv,
                             nn_buf q, nn_buf k, nn_buf v) {
    return linear_qkv(c, M, K, x, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v, nullptr, 0.f, "nn_linear_qkv");
}

extern "C" int nn_bias_add(nn_context* c, int rows, int cols, nn_buf out, nn_buf bias) {
    if (!c || !out || !bias) return NN_FAIL(NN_ERR_ARG, "nn_bias_add: null argument");
    if (rows < 0 || cols <= 0) return NN_FAIL(NN_ERR_ARG, "nn_bias_add: bad shape rows=%d cols=%d", rows, cols);
    if (rows == 0) return NN_OK;
    BiasArgs a = {};
    a.out[0] = (uint16_t*)out;
    a.bias[0] = (const uint16_t*)bias;
    a.cols[0] = cols;
    a.rows = rows;
    a.nseg = 1;
    ProfScope prof(c, "bias_add_rows" + std::to_string(rows) + "_cols" + std::to_string(cols));
    CUDA_TRY(launch_bias_add(a, c->stream));
    c->launches++;
    return NN_OK;
}

extern "C" int nn_linear_qkv_bias(nn_context* c, int M, int K, nn_buf x, nn_buf Wq, int Nq, nn_buf Wk, int Nk, nn_buf Wv, int Nv,
                                  nn_buf bq, nn_buf bk, nn_buf bv, nn_buf q, nn_buf k, nn_buf v) {
    if (!bq || !bk || !bv) return NN_FAIL(NN_ERR_ARG, "nn_linear_qkv_bias: null bias");
    return linear_qkv(c, M, K, x, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v, nullptr, 0.f, "nn_linear_qkv_bias", bq, bk, bv);
}

extern "C" int nn_rmsnorm(nn_context* c, int rows, int cols, nn_buf x, nn_buf weight, float eps, nn_buf out) {
    if (!c || !x || !weight || !out) return NN_FAIL(NN_ERR_ARG, "nn_rmsnorm: null argument");
    if (rows < 0 || cols <= 0) return NN_FAIL(NN_ERR_ARG, "nn_rmsnorm: bad shape rows=%d cols=%d", rows, cols);
    if (rows == 0) return NN_OK;
    ProfScope prof(c, "rmsnorm_rows" + std::to_string(rows) + "_cols" + std::to_string(cols));
    CUDA_TRY(launch_rmsnorm((const uint16_t*)x, (const uint16_t*)weight, (uint16_t*)out, rows, cols, eps, c->stream));
    c->launches++;
    return NN_OK;
}

extern "C" int nn_rmsnorm_linear(nn_context* c, int M, int N, int K, nn_buf x, nn_buf gamma, float eps, nn_buf W, nn_buf out) {
    if (!gamma) return NN_FAIL(NN_ERR_ARG, "nn_rmsnorm_linear: null norm weight");
    return one_weight(c, M, N, K, x, W, out, EPI_STORE, "nn_rmsnorm_linear", nullptr, 0, nullptr, gamma, eps);
}

extern "C" int nn_rmsnorm_linear_qkv(nn_context* c, int M, int K, nn_buf x, nn_buf gamma, float eps, nn_buf Wq, int Nq, nn_buf Wk, int Nk,
                                     nn_buf Wv, int Nv, nn_buf q, nn_buf k, nn_buf v) {
    if (!gamma) return NN_FAIL(NN_ERR_ARG, "nn_rmsnorm_linear_qkv: null norm weight");
    return linear_qkv(c, M, K, x, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v, gamma, eps, "nn_rmsnorm_linear_qkv");
}

extern "C" int nn_rmsnorm_linear_qkv_bias(nn_context* c, int M, int K, nn_buf x, nn_buf gamma, float eps, nn_buf Wq, int Nq, nn_buf Wk, int Nk,
                                          nn_buf Wv, int Nv, nn_buf bq, nn_buf bk, nn_buf bv, nn_buf q, nn_buf k, nn_buf v) {
    if (!gamma) return NN_FAIL(NN_ERR_ARG, "nn_rmsnorm_linear_qkv_bias: null norm weight");
    if (!bq || !bk || !bv) return NN_FAIL(NN_ERR_ARG, "nn_rmsnorm_linear_qkv_bias: null bias");
    return linear_qkv(c, M, K, x, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v, gamma, eps, "nn_rmsnorm_linear_qkv_bias", bq, bk, bv);
}

extern "C" int nn_rmsnorm_gate_up_silu(nn_context* c, int M, int N, int K, nn_buf x, nn_buf gamma, float eps, nn_buf Wg, nn_buf Wu, nn_buf out) {
    if (!gamma) return NN_FAIL(NN_ERR_ARG, "nn_rmsnorm_gate_up_silu: null norm weight");
    return gate_up_silu(c, M, N, K, x, Wg, Wu, out, gamma, eps, "nn_rmsnorm_gate_up_silu");
}

extern "C" int nn_dequant(nn_context* c, int N, int K, nn_buf W, nn_buf out) {
    if (!c || !W || !out) return NN_FAIL(NN_ERR_ARG, "nn_dequant: null argument");
    if (N <= 0 || K <= 0) return NN_FAIL(NN_ERR_ARG, "nn_dequant: bad shape N=%d K=%d", N, K);
    ResolvedW r;
    if (!resolve_weight(c, W, K, &r)) return NN_FAIL(NN_ERR_ARG, "nn_dequant: registration does not match K=%d", K);
    if (r.rows_avail >= 0 && N > r.rows_avail) return NN_FAIL(NN_ERR_ARG, "nn_dequant: N exceeds the registered rows");
    CUDA_TRY(launch_dequant(r.fmt, N, K, W, r.scale, (float*)out, c->stream));
    c->launches++;
    return NN_OK;
}

extern "C" int nn_linear_argmax(nn_context* c, int N, int K, nn_buf x, nn_buf W, nn_buf logits, nn_buf out_idx) {
    return nnb::linear_argmax(c, N, K, x, W, logits, out_idx, 0, nullptr, "nn_linear_argmax");
}

int nnb::linear_argmax(nn_context* c, int N, int K, nn_buf x, nn_buf W, nn_buf logits, nn_buf out_idx, int row_base, const GatherSignal* sig,
                       const char* who) {
    int rc = check_common(c, 1, N, K, x, W, out_idx, who);
    if (rc) return rc;
    ResolvedW r;
    if (!resolve_weight(c, W, K, &r))
        return NN_FAIL(NN_ERR_ARG, "%s: W points into a registered quantised weight but K=%d or the row offset does not match", who, K);
    if (r.rows_avail >= 0 && N > r.rows_avail)
        return NN_FAIL(NN_ERR_ARG, "%s: N=%d exceeds the %d rows registered for this weight", who, N, r.rows_avail);
    LinArgs a = {};
    a.nseg = 1;
    a.seg[0].W = (const uint8_t*)W;
    a.seg[0].scale = r.scale;
    a.scale_pad[0] = r.scale_pad;
    a.scale_pitch = r.scale_pitch;
    a.seg[0].out = (uint16_t*)logits;
    a.seg[0].N = N;
    a.seg[0].ld_out = N;
    a.x = (const uint16_t*)x;
    a.M = 1;
    a.K = K;
    a.epi = EPI_STORE;
    a.status = c->status_dev;
    a.sk_scratch = c->sk_scratch;
    a.sk_flags = c->sk_flags;
    StreamPlan p = {};
    if (stream_supported(r.fmt, 1, K, a)) p = stream_plan(r.fmt, a, c->sm_count, c->smem_limit);
    if (!p.ok) {
        // shapes the streaming kernel does not take: projection, then the separate arg-max
        if (sig) return NN_FAIL(NN_ERR_UNSUPPORTED, "%s: this shape (K=%d) is not taken by the streaming kernel", who, K);
        if (!logits) return NN_FAIL(NN_ERR_UNSUPPORTED, "%s: this shape (K=%d) needs a logits buffer", who, K);
        rc = one_weight(c, 1, N, K, x, W, logits, EPI_STORE, who);
        if (rc) return rc;
        return nn_argmax(c, N, logits, out_idx);
    }
    ProfScope prof(c, op_label(1, N, K, r.fmt, "_argmax"));
    a.argmax_slot = c->argmax_slot + 1;
    a.argmax_done = reinterpret_cast<unsigned*>(c->argmax_slot + 2);
    a.argmax_out = (int*)out_idx;
    a.argmax_base = row_base;
    if (sig) a.sig = *sig;
    cudaError_t e = launch_stream(r.fmt, a, p, c->stream, c->use_pdl);
    if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "%s: launch failed: %s (N=%d K=%d)", who, cudaGetErrorString(e), N, K);
    note_recorded(c, r.fmt, a, p);
    c->launches++;
    return NN_OK;
}

extern "C" int nn_argmax(nn_context* c, int n, nn_buf logits, nn_buf out_idx) {
    if (!c || !logits || !out_idx) return NN_FAIL(NN_ERR_ARG, "nn_argmax: null argument");
    if (n < 0) return NN_FAIL(NN_ERR_ARG, "nn_argmax: n=%d", n);
    ProfScope prof(c, "argmax_n" + std::to_string(n));
    CUDA_TRY(launch_argmax_half((const uint16_t*)logits, n, (int*)out_idx, c->argmax_slot, c->stream));
    c->launches += n > 0 ? 3 : 2;
    return NN_OK;
}

// ---------------------------------------------------------------------------------
// recorded decode step.  The operator calls between nn_plan_begin and nn_plan_end are captured
// into a CUDA graph (programmatic-launch edges kept).  Runs of consecutive single-token
// streaming operators inside it are then replaced by one launch each of the resident kernel
// (decode_plan.cu); whatever else was recorded on the stream in between (other library
// kernels, the caller's own kernels and copies) stays where it is, as the node it was.
// ---------------------------------------------------------------------------------
struct nn_plan {
    int device = 0;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int kernels = 0;      // launches per replay
    int recorded = 0;     // launches that were recorded
    std::vector<PlanRun> runs;
    std::vector<cudaGraphNode_t> run_nodes;  // the graph node of each run
};

extern "C" int nn_plan_begin(nn_context* c) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "nn_plan_begin: null context");
    if (c->capturing) return NN_FAIL(NN_ERR_ARG, "nn_plan_begin: already recording");
    CUDA_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    c->capturing = true;
    c->rec.clear();
    c->launches_at_capture = c->launches;
    return NN_OK;
}

static HazardOp hazard_view(const RecordedOp& r) {
    HazardOp h;
    const LinArgs& a = r.a;
    h.x = (uintptr_t)a.x;
    h.x_bytes = (size_t)a.K * 2;
    for (int k = 0; k < a.nseg; ++k)
        if (a.seg[k].out) {
            h.out[h.nout] = (uintptr_t)a.seg[k].out;
            h.out_bytes[h.nout] = (size_t)a.seg[k].N * 2;
            h.nout++;
        }
    h.inplace = a.epi == EPI_RESIDUAL || a.epi == EPI_SILU_GATE;
    if (a.argmax_slot) {
        h.has_argmax = true;
        h.out[h.nout] = (uintptr_t)a.argmax_out;
        h.out_bytes[h.nout] = 4;
        h.nout++;
    }
    return h;
}

static void set_run_node_params(cudaGraphNode_t node, PlanRun& run, cudaError_t* err) {
    const void* fn = nullptr;
    decode_plan_func(&fn);
    cudaKernelNodeParams kp = {};
    kp.func = const_cast<void*>(fn);
    kp.gridDim = dim3((unsigned)run.grid);
    kp.blockDim = dim3((unsigned)DECODE_PLAN_THREADS);
    kp.sharedMemBytes = (unsigned)run.smem;
    void* args[1] = {&run.params};
    kp.kernelParams = args;
    kp.extra = nullptr;
    *err = cudaGraphKernelNodeSetParams(node, &kp);
}

// Replace runs of recorded streaming operators by resident launches, on a clone of the captured
// graph; any failure leaves the captured graph as it was.  Returns the graph to instantiate.
static cudaGraph_t consolidate_runs(nn_context* c, nn_plan* p, cudaGraph_t g) {
    const std::vector<RecordedOp>& rec = c->rec;
    if (rec.size() < 2 || getenv("NNB_PLAN_SEPARATE")) return g;
    // the capture of one stream is a chain: successor of every node
    size_t ne = 0;
    if (cudaGraphGetEdges_v2(g, nullptr, nullptr, nullptr, &ne) != cudaSuccess) return g;
    std::vector<cudaGraphNode_t> from(ne), to(ne);
    std::vector<cudaGraphEdgeData> ed(ne);
    if (ne && cudaGraphGetEdges_v2(g, from.data(), to.data(), ed.data(), &ne) != cudaSuccess) return g;
    std::map<cudaGraphNode_t, cudaGraphNode_t> succ;
    std::map<cudaGraphNode_t, int> npred;
    for (size_t i = 0; i < ne; ++i) {
        if (succ.count(from[i])) return g;  // a fork: not a simple chain
        succ[from[i]] = to[i];
        if (++npred[to[i]] > 1) return g;   // a join
    }
    std::vector<HazardOp> hz(rec.size());
    for (size_t i = 0; i < rec.size(); ++i) hz[i] = hazard_view(rec[i]);
    // bias rows are read like weights, with no ordering of their own: an operator whose bias any recorded operator writes
    // keeps its own launch
    std::vector<char> elig(rec.size());
    for (size_t i = 0; i < rec.size(); ++i) {
        elig[i] = rec[i].eligible ? 1 : 0;
        for (int k = 0; k < rec[i].a.nseg && elig[i]; ++k) {
            const uint16_t* bp = rec[i].a.seg[k].bias;
            if (!bp) continue;
            const uintptr_t b0 = (uintptr_t)bp, b1 = b0 + (size_t)rec[i].a.seg[k].N * 2;
            for (size_t j = 0; j < rec.size() && elig[i]; ++j)
                for (int o = 0; o < hz[j].nout; ++o)
                    if (b0 < hz[j].out[o] + hz[j].out_bytes[o] && hz[j].out[o] < b1) elig[i] = 0;
        }
    }
    cudaGraph_t g2 = nullptr;
    if (cudaGraphClone(&g2, g) != cudaSuccess) return g;
    auto give_up = [&]() {
        for (PlanRun& r : p->runs) free_run(&r);
        p->runs.clear();
        p->run_nodes.clear();
        cudaGraphDestroy(g2);
        return g;
    };
    cudaSetDevice(c->device);
    int removed = 0;
    size_t i = 0;
    while (i < rec.size()) {
        if (!elig[i]) { ++i; continue; }
        // operators that follow one another directly in the graph
        size_t j = i + 1;
        while (j < rec.size() && elig[j] && succ.count(rec[j - 1].node) && succ[rec[j - 1].node] == rec[j].node) ++j;
        // [i, j) is a candidate; the data hazards may cut it shorter
        std::vector<HazardOp> cand(hz.begin() + i, hz.begin() + j);
        std::vector<OpDeps> deps;
        const int len = analyze_run(cand, 0, &deps);
        if (len < 2) { ++i; continue; }
        PlanRun run;
        const char* why = "";
        cudaError_t e = build_run(rec, deps, (int)i, len, c->sm_count, c->smem_limit, c->status_dev, &run, &why);
        if (e != cudaSuccess) {
            free_run(&run);
            cudaGetLastError();
            i += len;  // these operators stay separate launches
            continue;
        }
        p->runs.push_back(run);
        PlanRun& kept = p->runs.back();
        // the run's first node becomes the resident launch; the others leave the graph
        cudaGraphNode_t head = nullptr;
        if (cudaGraphNodeFindInClone(&head, rec[i].node, g2) != cudaSuccess) return give_up();
        set_run_node_params(head, kept, &e);
        if (e != cudaSuccess) return give_up();
        cudaGraphNode_t after = nullptr;
        const cudaGraphNode_t last = rec[i + len - 1].node;
        if (succ.count(last) && cudaGraphNodeFindInClone(&after, succ[last], g2) != cudaSuccess) return give_up();
        for (int k = 1; k < len; ++k) {
            cudaGraphNode_t n2 = nullptr;
            if (cudaGraphNodeFindInClone(&n2, rec[i + k].node, g2) != cudaSuccess || cudaGraphDestroyNode(n2) != cudaSuccess) return give_up();
        }
        if (after && cudaGraphAddDependencies(g2, &head, &after, 1) != cudaSuccess) return give_up();
        p->run_nodes.push_back(head);
        removed += len - 1;
        i += len;
    }
    if (p->runs.empty()) {
        cudaGraphDestroy(g2);
        return g;
    }
    // run.params was copied into the node when it was set; p->runs keeps the device tables alive
    cudaGraphExec_t probe = nullptr;
    if (cudaGraphInstantiate(&probe, g2, 0) != cudaSuccess) {
        cudaGetLastError();
        return give_up();
    }
    p->exec = probe;
    p->kernels -= removed;
    cudaGraphDestroy(g);
    return g2;
}

extern "C" int nn_plan_end(nn_context* c, nn_plan** out) {
    if (!c || !out) return NN_FAIL(NN_ERR_ARG, "nn_plan_end: null argument");
    if (!c->capturing) return NN_FAIL(NN_ERR_ARG, "nn_plan_end: not recording");
    c->capturing = false;
    nn_plan* p = new nn_plan();
    p->device = c->device;
    cudaError_t e = cudaStreamEndCapture(c->stream, &p->graph);
    if (e != cudaSuccess || !p->graph) {
        delete p;
        c->rec.clear();
        return NN_FAIL(NN_ERR_CUDA, "nn_plan_end: capture failed: %s", cudaGetErrorString(e));
    }
    p->recorded = p->kernels = (int)(c->launches - c->launches_at_capture);
    c->launches = c->launches_at_capture;  // recorded, not run
    p->graph = consolidate_runs(c, p, p->graph);
    c->rec.clear();
    if (!p->exec) {
        e = cudaGraphInstantiate(&p->exec, p->graph, 0);
        if (e != cudaSuccess) {
            cudaGraphDestroy(p->graph);
            delete p;
            return NN_FAIL(NN_ERR_CUDA, "nn_plan_end: instantiate failed: %s", cudaGetErrorString(e));
        }
    }
    *out = p;
    return NN_OK;
}

extern "C" int nn_plan_launch(nn_context* c, nn_plan* p) {
    if (!c || !p || !p->exec) return NN_FAIL(NN_ERR_ARG, "nn_plan_launch: null argument");
    ProfScope prof(c, "plan_replay_" + std::to_string(p->recorded) + "ops_" + std::to_string(p->kernels) + "launches");
    CUDA_TRY(cudaGraphLaunch(p->exec, c->stream));
    c->launches += p->kernels;
    return NN_OK;
}

extern "C" int nn_plan_num_kernels(const nn_plan* p) { return p ? p->kernels : 0; }
extern "C" int nn_plan_num_recorded(const nn_plan* p) { return p ? p->recorded : 0; }
extern "C" int nn_plan_num_resident_runs(const nn_plan* p) { return p ? (int)p->runs.size() : 0; }

extern "C" int nn_plan_set_wait_limit(nn_plan* p, unsigned timeout_ms) {
    if (!p || !p->exec) return NN_FAIL(NN_ERR_ARG, "nn_plan_set_wait_limit: null plan");
    if (timeout_ms < 1 || timeout_ms > 10000) return NN_FAIL(NN_ERR_ARG, "nn_plan_set_wait_limit: %u ms is outside [1, 10000]", timeout_ms);
    for (size_t i = 0; i < p->runs.size(); ++i) {
        p->runs[i].params.wait_cycles = (long long)timeout_ms * 2000000ll;  // at most 2 GHz
        cudaError_t e;
        set_run_node_params(p->run_nodes[i], p->runs[i], &e);
        if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "nn_plan_set_wait_limit: %s", cudaGetErrorString(e));
    }
    if (!p->runs.empty()) {
        cudaGraphExec_t ex = nullptr;
        CUDA_TRY(cudaGraphInstantiate(&ex, p->graph, 0));
        cudaGraphExecDestroy(p->exec);
        p->exec = ex;
    }
    return NN_OK;
}

extern "C" int nn_plan_withhold_output(nn_plan* p, int run_index, int op_index) {
    if (!p || !p->exec) return NN_FAIL(NN_ERR_ARG, "nn_plan_withhold_output: null plan");
    if (run_index < 0 || run_index >= (int)p->runs.size()) return NN_FAIL(NN_ERR_ARG, "nn_plan_withhold_output: the plan has %zu resident runs", p->runs.size());
    PlanRun& r = p->runs[run_index];
    if (op_index < -1 || op_index >= r.count) return NN_FAIL(NN_ERR_ARG, "nn_plan_withhold_output: run %d has %d operators", run_index, r.count);
    r.params.drop_publish_op = op_index;
    cudaError_t e;
    set_run_node_params(p->run_nodes[run_index], r, &e);
    if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "nn_plan_withhold_output: %s", cudaGetErrorString(e));
    cudaGraphExec_t ex = nullptr;
    CUDA_TRY(cudaGraphInstantiate(&ex, p->graph, 0));
    cudaGraphExecDestroy(p->exec);
    p->exec = ex;
    return NN_OK;
}

extern "C" int nn_plan_analyze(int nops, const uint64_t* x_addr, const uint64_t* x_bytes, const uint64_t* out_addr, const uint64_t* out_bytes,
                               const int* nout, const int* flags, int first, int* x_dep, int* res_dep, int* store_mask, int* publish_mask) {
    if (nops < 0 || first < 0 || first > nops || (nops && (!x_addr || !x_bytes || !out_addr || !out_bytes || !nout || !flags)))
        return NN_FAIL(NN_ERR_ARG, "nn_plan_analyze: bad argument");
    std::vector<HazardOp> ops((size_t)nops);
    for (int i = 0; i < nops; ++i) {
        if (nout[i] < 0 || nout[i] > 4) return NN_FAIL(NN_ERR_ARG, "nn_plan_analyze: operator %d has %d outputs", i, nout[i]);
        ops[i].x = (uintptr_t)x_addr[i];
        ops[i].x_bytes = (size_t)x_bytes[i];
        ops[i].nout = nout[i];
        for (int k = 0; k < nout[i]; ++k) {
            ops[i].out[k] = (uintptr_t)out_addr[4 * i + k];
            ops[i].out_bytes[k] = (size_t)out_bytes[4 * i + k];
        }
        ops[i].inplace = (flags[i] & 1) != 0;
        ops[i].has_argmax = (flags[i] & 2) != 0;
    }
    std::vector<OpDeps> deps;
    const int len = analyze_run(ops, first, &deps);
    for (int i = 0; i < len; ++i) {
        if (x_dep) x_dep[i] = deps[i].x_dep;
        if (res_dep) res_dep[i] = deps[i].res_dep;
        int sm = 0, pm = 0;
        const int nweights = ops[first + i].nout - (ops[first + i].has_argmax ? 1 : 0);
        for (int k = 0; k < 3 && k < nweights; ++k) {
            if (deps[i].store[k]) sm |= 1 << k;
            if (deps[i].publish[k]) pm |= 1 << k;
        }
        if (store_mask) store_mask[i] = sm;
        if (publish_mask) publish_mask[i] = pm;
    }
    return len;
}

extern "C" int nn_plan_free(nn_plan* p) {
    if (!p) return NN_OK;
    cudaSetDevice(p->device);
    if (p->exec) cudaGraphExecDestroy(p->exec);
    if (p->graph) cudaGraphDestroy(p->graph);
    for (PlanRun& r : p->runs) free_run(&r);
    delete p;
    return NN_OK;
}

// ---------------------------------------------------------------------------------
// timing
// ---------------------------------------------------------------------------------
extern "C" int nn_event_create(void** out) {
    if (!out) return NN_FAIL(NN_ERR_ARG, "nn_event_create: null argument");
    cudaEvent_t ev;
    CUDA_TRY(cudaEventCreate(&ev));
    *out = (void*)ev;
    return NN_OK;
}
extern "C" int nn_event_record(nn_context* c, void* ev) {
    if (!c || !ev) return NN_FAIL(NN_ERR_ARG, "nn_event_record: null argument");
    CUDA_TRY(cudaEventRecord((cudaEvent_t)ev, c->stream));
    return NN_OK;
}
extern "C" int nn_event_elapsed_ms(void* a, void* b, float* ms) {
    if (!a || !b || !ms) return NN_FAIL(NN_ERR_ARG, "nn_event_elapsed_ms: null argument");
    CUDA_TRY(cudaEventSynchronize((cudaEvent_t)b));
    CUDA_TRY(cudaEventElapsedTime(ms, (cudaEvent_t)a, (cudaEvent_t)b));
    return NN_OK;
}
extern "C" int nn_event_destroy(void* ev) {
    if (ev) CUDA_TRY(cudaEventDestroy((cudaEvent_t)ev));
    return NN_OK;
}

extern "C" int nn_bandwidth_probe(nn_context* c, size_t bytes, int trials, double* out_loads_gbs, double* out_tma_gbs) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "nn_bandwidth_probe: null context");
    if (c->capturing) return NN_FAIL(NN_ERR_UNSUPPORTED, "nn_bandwidth_probe: not inside a recording");
    if (bytes == 0) bytes = c->l2_bytes * 8 > ((size_t)1 << 30) ? c->l2_bytes * 8 : ((size_t)1 << 30);
    bytes &= ~(size_t)16383;
    if (bytes < ((size_t)1 << 20) || trials < 1 || trials > 100)
        return NN_FAIL(NN_ERR_ARG, "nn_bandwidth_probe: bytes=%zu (at least 1 MiB) trials=%d (1..100)", bytes, trials);
    cudaSetDevice(c->device);
    uint8_t* src = nullptr;
    float* sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = NN_OK;
    double best[2] = {0, 0};
    auto fail = [&](cudaError_t e, const char* what) { rc = NN_FAIL(NN_ERR_CUDA, "nn_bandwidth_probe: %s: %s", what, cudaGetErrorString(e)); };
    cudaError_t e = cudaMalloc((void**)&src, bytes);
    if (e != cudaSuccess) { fail(e, "cudaMalloc"); return rc; }
    if ((e = cudaMalloc((void**)&sink, 2048)) != cudaSuccess) fail(e, "cudaMalloc");
    if (!rc && (e = cudaMemsetAsync(src, 0x3c, bytes, c->stream)) != cudaSuccess) fail(e, "cudaMemsetAsync");
    if (!rc && (e = cudaMemsetAsync(sink, 0, 2048, c->stream)) != cudaSuccess) fail(e, "cudaMemsetAsync");
    if (!rc && ((e = cudaEventCreate(&e0)) != cudaSuccess || (e = cudaEventCreate(&e1)) != cudaSuccess)) fail(e, "cudaEventCreate");
    unsigned* status = reinterpret_cast<unsigned*>(sink + 256);
    for (int path = 0; path < 2 && !rc; ++path) {
        for (int t = 0; t < trials && !rc; ++t) {
            for (int rep = 0; rep < 2 && !rc; ++rep) {  // one untimed, one timed: the buffer is larger than L2, nothing of it stays
                if (rep) cudaEventRecord(e0, c->stream);
                e = path == 0 ? launch_probe_loads(src, bytes, sink, c->stream) : launch_probe_tma(src, bytes, status, c->stream);
                if (e != cudaSuccess) fail(e, "launch");
                c->launches++;
            }
            if (rc) break;
            cudaEventRecord(e1, c->stream);
            if ((e = cudaEventSynchronize(e1)) != cudaSuccess) { fail(e, "cudaEventSynchronize"); break; }
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            const double gbs = ms > 0 ? (double)bytes / (ms * 1e-3) / 1e9 : 0.0;
            if (gbs > best[path]) best[path] = gbs;
        }
    }
    if (!rc) {
        unsigned st = 0;
        if ((e = cudaMemcpy(&st, status, sizeof(st), cudaMemcpyDeviceToHost)) != cudaSuccess) fail(e, "cudaMemcpy");
        else if (st) rc = NN_FAIL(NN_ERR_TIMEOUT, "nn_bandwidth_probe: a bulk copy did not land within the wait limit");
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(sink);
    cudaFree(src);
    if (rc) return rc;
    if (out_loads_gbs) *out_loads_gbs = best[0];
    if (out_tma_gbs) *out_tma_gbs = best[1];
    return NN_OK;
}

extern "C" int nn_l2_flush(nn_context* c) {
    if (!c) return NN_FAIL(NN_ERR_ARG, "nn_l2_flush: null context");
    if (!c->flush_buf) {
        c->flush_bytes = c->l2_bytes * 2 > ((size_t)256 << 20) ? c->l2_bytes * 2 : ((size_t)256 << 20);
        cudaSetDevice(c->device);
        CUDA_TRY(cudaMalloc(&c->flush_buf, c->flush_bytes));
        CUDA_TRY(cudaMemsetAsync(c->flush_buf, 0, c->flush_bytes, c->stream));
    }
    CUDA_TRY(launch_l2_flush(c->flush_buf, c->flush_bytes, c->stream));
    return NN_OK;
}
