// Row-sharding communicator: one rank per GPU, NCCL all-gather of the per-rank
// [M, N/G] output blocks over NVLink / NVSwitch.  The reference is single-device;
// this extends its row tiling of large weights (src/models/lfm2-5-350m/src/utils.cpp:427-452:
// sub-buffers of W, scale and out by row range) from image tiles to ranks.
//
// NCCL is resolved at run time with dlopen so that the single-GPU library has no
// link-time dependency on it.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/nnopt_b200.h"
#include "internal.h"
#include "kernels.h"

namespace {

struct NcclId { char bytes[128]; };
typedef int (*fn_get_unique_id)(NcclId*);
typedef int (*fn_comm_init_rank)(void**, int, NcclId, int);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*fn_comm_destroy)(void*);
typedef const char* (*fn_error_string)(int);

struct NcclApi {
    void* handle = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_error_string error_string = nullptr;
    bool tried = false;
};
NcclApi g_nccl;

bool load_nccl() {
    if (g_nccl.tried) return g_nccl.handle != nullptr;
    g_nccl.tried = true;
    // NNB_NCCL_LIB, when set, names the only library tried: a wrong path is an error, never a
    // silent switch to whatever libnccl the loader finds
    const char* forced = getenv("NNB_NCCL_LIB");
    void* h = nullptr;
    if (forced && forced[0]) {
        h = dlopen(forced, RTLD_NOW | RTLD_GLOBAL);
    } else {
        const char* names[2] = {"libnccl.so.2", "libnccl.so"};
        for (int i = 0; i < 2 && !h; ++i) h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    }
    if (!h) return false;
    g_nccl.get_unique_id = (fn_get_unique_id)dlsym(h, "ncclGetUniqueId");
    g_nccl.comm_init_rank = (fn_comm_init_rank)dlsym(h, "ncclCommInitRank");
    g_nccl.all_gather = (fn_all_gather)dlsym(h, "ncclAllGather");
    g_nccl.comm_destroy = (fn_comm_destroy)dlsym(h, "ncclCommDestroy");
    g_nccl.error_string = (fn_error_string)dlsym(h, "ncclGetErrorString");
    if (!g_nccl.get_unique_id || !g_nccl.comm_init_rank || !g_nccl.all_gather || !g_nccl.comm_destroy) {
        dlclose(h);
        return false;
    }
    g_nccl.handle = h;
    return true;
}

const char* nccl_err(int rc) { return g_nccl.error_string ? g_nccl.error_string(rc) : "nccl error"; }

}  // namespace

// One buffer of the same size on every rank, each rank holding peer mappings of the others'.
struct SymmAlloc {
    void* base[8] = {};  // base[rank] is this rank's own allocation, the rest are peer mappings
    size_t bytes = 0;
};

struct nn_comm {
    nn_context* ctx = nullptr;
    void* comm = nullptr;
    int rank = 0, world = 1;
    std::vector<SymmAlloc> symm;
    unsigned* flags = nullptr;   // symmetric: word g is written by rank g's signal kernel
    unsigned* epochs = nullptr;  // local: [0] signals sent, [1] waits done, [2] blocks done, [3] picks sent, [4] picks waited,
                                 // [5] batched picks done
    int row_keys = -1;           // index in symm of the batched pick's key tables, allocated on first use
};

#define COMM_CUDA(call)                                                                                   \
    do {                                                                                                  \
        cudaError_t e_ = (call);                                                                          \
        if (e_ != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_));      \
    } while (0)

namespace {

// Allocates `bytes` on this rank, exchanges CUDA IPC handles through the communicator and maps the
// other ranks' allocations.  Collective: every rank calls it with the same size, in the same order.
// The allocation is rounded up to whole 2 MiB pages: an exported IPC handle opens the allocation's whole
// page range on the peers, and nothing else of this process may live there.
int symm_alloc(nn_comm* c, size_t bytes, SymmAlloc* out) {
    SymmAlloc sa;
    sa.bytes = bytes;
    cudaSetDevice(c->ctx->device);
    const size_t page = (size_t)2 << 20;
    const size_t padded = (bytes + page - 1) / page * page;
    void* local = nullptr;
    void* dev = nullptr;  // staging for the handle exchange
    auto fail = [&](int rc) {
        for (int g = 0; g < c->world; ++g)
            if (g != c->rank && sa.base[g]) cudaIpcCloseMemHandle(sa.base[g]);
        if (dev) cudaFree(dev);
        if (local) cudaFree(local);
        return rc;
    };
#define SYMM_CUDA(call)                                                                                         \
    do {                                                                                                        \
        cudaError_t e_ = (call);                                                                                \
        if (e_ != cudaSuccess) return fail(NN_FAIL(NN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)));      \
    } while (0)
    SYMM_CUDA(cudaMalloc(&local, padded));
    SYMM_CUDA(cudaMemsetAsync(local, 0, padded, c->ctx->stream));
    if (c->world > 1) {
        cudaIpcMemHandle_t mine;
        SYMM_CUDA(cudaIpcGetMemHandle(&mine, local));
        const size_t hb = sizeof(cudaIpcMemHandle_t);
        std::vector<cudaIpcMemHandle_t> all((size_t)c->world);
        SYMM_CUDA(cudaMalloc(&dev, hb * c->world));
        SYMM_CUDA(cudaMemcpyAsync((char*)dev + hb * c->rank, &mine, hb, cudaMemcpyHostToDevice, c->ctx->stream));
        const int rc = g_nccl.all_gather((char*)dev + hb * c->rank, dev, hb, /*ncclInt8*/ 0, c->comm, c->ctx->stream);
        if (rc != 0) return fail(NN_FAIL(NN_ERR_COMM, "ncclAllGather (handle exchange): %s", nccl_err(rc)));
        SYMM_CUDA(cudaMemcpyAsync(all.data(), dev, hb * c->world, cudaMemcpyDeviceToHost, c->ctx->stream));
        SYMM_CUDA(cudaStreamSynchronize(c->ctx->stream));
        cudaFree(dev);
        dev = nullptr;
        for (int g = 0; g < c->world; ++g) {
            if (g == c->rank) continue;
            void* p = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&p, all[(size_t)g], cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess)
                return fail(NN_FAIL(NN_ERR_COMM, "rank %d cannot map rank %d's buffer (cudaIpcOpenMemHandle: %s); peer access is required",
                                    c->rank, g, cudaGetErrorString(e)));
            sa.base[g] = p;
        }
    } else {
        SYMM_CUDA(cudaStreamSynchronize(c->ctx->stream));
    }
#undef SYMM_CUDA
    sa.base[c->rank] = local;
    *out = sa;
    return NN_OK;
}

// Releasing is collective and has two phases with a barrier between them: first every rank closes
// its mappings of the others' buffers, then, once all ranks have done so, each frees its own (freeing
// memory that a peer still has open through an IPC handle is undefined).
void symm_close_peers(nn_comm* c, SymmAlloc& sa) {
    for (int g = 0; g < c->world; ++g) {
        if (g == c->rank || !sa.base[g]) continue;
        cudaIpcCloseMemHandle(sa.base[g]);
        sa.base[g] = nullptr;
    }
}
void ranks_barrier(nn_comm* c) {
    if (c->world <= 1 || !c->comm || !c->epochs) return;
    // one byte per rank through the communicator, then a host wait: every rank has reached this point
    char* scratch = reinterpret_cast<char*>(c->epochs) + 32;
    if (g_nccl.all_gather(scratch + c->rank, scratch, 1, /*ncclInt8*/ 0, c->comm, c->ctx->stream) == 0) cudaStreamSynchronize(c->ctx->stream);
}
void symm_free_local(nn_comm* c, SymmAlloc& sa) {
    if (sa.base[c->rank]) cudaFree(sa.base[c->rank]);
    sa.base[c->rank] = nullptr;
}

}  // namespace

extern "C" int nn_comm_unique_id(void* out) {
    if (!out) return NN_FAIL(NN_ERR_ARG, "nn_comm_unique_id: null argument");
    if (!load_nccl()) {
        const char* why = dlerror();
        return NN_FAIL(NN_ERR_COMM, "NCCL could not be loaded (NNB_NCCL_LIB names the library to use, default libnccl.so.2): %s",
                       why ? why : "see the first failure");
    }
    NcclId id;
    const int rc = g_nccl.get_unique_id(&id);
    if (rc != 0) return NN_FAIL(NN_ERR_COMM, "ncclGetUniqueId: %s", nccl_err(rc));
    memcpy(out, id.bytes, sizeof(id.bytes));
    return NN_OK;
}

extern "C" int nn_comm_init(nn_context* ctx, const void* id_bytes, int rank, int world, nn_comm** out) {
    if (!ctx || !out) return NN_FAIL(NN_ERR_ARG, "nn_comm_init: null argument");
    if (world < 1 || rank < 0 || rank >= world) return NN_FAIL(NN_ERR_ARG, "nn_comm_init: rank %d of %d", rank, world);
    *out = nullptr;
    nn_comm* c = new nn_comm();
    c->ctx = ctx;
    c->rank = rank;
    c->world = world;
    if (world > 1) {
        if (!id_bytes) { delete c; return NN_FAIL(NN_ERR_ARG, "nn_comm_init: null unique id"); }
        if (!load_nccl()) { delete c; return NN_FAIL(NN_ERR_COMM, "NCCL could not be loaded (NNB_NCCL_LIB names the library to use, default libnccl.so.2)"); }
        NcclId id;
        memcpy(id.bytes, id_bytes, sizeof(id.bytes));
        cudaSetDevice(ctx->device);
        const int rc = g_nccl.comm_init_rank(&c->comm, world, id, rank);
        if (rc != 0) { delete c; return NN_FAIL(NN_ERR_COMM, "ncclCommInitRank: %s", nccl_err(rc)); }
    }
    *out = c;
    return NN_OK;
}

extern "C" int nn_comm_symm_alloc(nn_comm* c, size_t bytes, nn_buf* out) {
    if (!c || !out || bytes == 0) return NN_FAIL(NN_ERR_ARG, "nn_comm_symm_alloc: null argument or zero size");
    *out = nullptr;
    if (c->world > 8) return NN_FAIL(NN_ERR_UNSUPPORTED, "nn_comm_symm_alloc: at most 8 ranks (one NVSwitch domain)");
    if (!c->flags) {
        // first use: the flag words (symmetric) and the two local epoch counters
        SymmAlloc fl;
        int rc = symm_alloc(c, 256, &fl);
        if (rc) return rc;
        c->symm.push_back(fl);
        c->flags = (unsigned*)fl.base[c->rank];
        COMM_CUDA(cudaMalloc((void**)&c->epochs, 64));
        COMM_CUDA(cudaMemset(c->epochs, 0, 64));
    }
    SymmAlloc sa;
    int rc = symm_alloc(c, bytes, &sa);
    if (rc) return rc;
    c->symm.push_back(sa);
    *out = sa.base[c->rank];
    return NN_OK;
}

extern "C" int nn_comm_symm_free(nn_comm* c, nn_buf buf) {
    if (!c || !buf) return NN_OK;
    for (size_t i = 0; i < c->symm.size(); ++i)
        if (c->symm[i].base[c->rank] == buf && buf != (void*)c->flags) {
            cudaSetDevice(c->ctx->device);
            cudaStreamSynchronize(c->ctx->stream);
            symm_close_peers(c, c->symm[i]);
            ranks_barrier(c);
            symm_free_local(c, c->symm[i]);
            c->symm.erase(c->symm.begin() + (long)i);
            return NN_OK;
        }
    return NN_FAIL(NN_ERR_ARG, "nn_comm_symm_free: %p is not a symmetric buffer of this communicator", buf);
}

extern "C" int nn_comm_signal(nn_comm* c) {
    if (!c || !c->flags) return NN_FAIL(NN_ERR_ARG, "nn_comm_signal: no symmetric buffer has been allocated on this communicator");
    nnb::PeerFlags pf = {};
    pf.world = c->world;
    pf.rank = c->rank;
    for (int g = 0; g < c->world; ++g) pf.flags[g] = (unsigned*)c->symm[0].base[g];
    COMM_CUDA(nnb::launch_comm_signal(pf, c->epochs, c->ctx->stream));
    c->ctx->launches++;
    return NN_OK;
}

extern "C" int nn_comm_wait(nn_comm* c, unsigned timeout_ms) {
    if (!c || !c->flags) return NN_FAIL(NN_ERR_ARG, "nn_comm_wait: no symmetric buffer has been allocated on this communicator");
    if (timeout_ms == 0 || timeout_ms > 10000) return NN_FAIL(NN_ERR_ARG, "nn_comm_wait: timeout %u ms outside 1..10000", timeout_ms);
    COMM_CUDA(nnb::launch_comm_wait(c->flags, c->world, c->epochs + 1, timeout_ms, c->ctx->status_dev, false, c->ctx->stream));
    c->ctx->launches++;
    return NN_OK;
}

extern "C" int nn_linear_gather(nn_comm* c, int M, int n_local, int K, nn_buf x, nn_buf W, nn_buf gathered) {
    if (!c || !gathered) return NN_FAIL(NN_ERR_ARG, "nn_linear_gather: null argument");
    if (M <= 0 || n_local <= 0) return NN_FAIL(NN_ERR_ARG, "nn_linear_gather: bad shape M=%d n_local=%d", M, n_local);
    const SymmAlloc* sa = nullptr;
    for (const SymmAlloc& s : c->symm)
        if (s.base[c->rank] == gathered) sa = &s;
    if (!sa) return NN_FAIL(NN_ERR_ARG, "nn_linear_gather: %p was not returned by nn_comm_symm_alloc on this communicator", gathered);
    const size_t block = (size_t)M * n_local * 2;
    if (block * c->world > sa->bytes)
        return NN_FAIL(NN_ERR_ARG, "nn_linear_gather: %d blocks of %zu bytes exceed the %zu-byte gather buffer", c->world, block, sa->bytes);
    uint16_t* peers[7];
    int np = 0;
    for (int g = 0; g < c->world; ++g)
        if (g != c->rank) peers[np++] = (uint16_t*)((char*)sa->base[g] + block * c->rank);
    // the projection kernel's last block sends this rank's signal; the wait kernel is launched
    // so that it is already spinning when that happens
    nnb::GatherSignal sig = {};
    sig.world = c->world;
    sig.rank = c->rank;
    for (int g = 0; g < c->world; ++g) sig.flags[g] = (unsigned*)c->symm[0].base[g];
    sig.epoch = c->epochs;
    sig.done = c->epochs + 2;
    int rc = nnb::linear_to_peers(c->ctx, M, n_local, K, x, W, (char*)gathered + block * c->rank, peers, np, &sig, "nn_linear_gather");
    if (rc) return rc;
    COMM_CUDA(nnb::launch_comm_wait(c->flags, c->world, c->epochs + 1, 2000, c->ctx->status_dev, c->ctx->use_pdl, c->ctx->stream));
    c->ctx->launches++;
    return NN_OK;
}

extern "C" int nn_linear_argmax_sharded(nn_comm* c, int n_local, int K, nn_buf x, nn_buf W, nn_buf logits_local, nn_buf out_idx) {
    const char* who = "nn_linear_argmax_sharded";
    if (!c || !out_idx) return NN_FAIL(NN_ERR_ARG, "%s: null argument", who);
    if (!c->flags) return NN_FAIL(NN_ERR_ARG, "%s: no symmetric buffer has been allocated on this communicator", who);
    if (n_local <= 0 || (long long)n_local * c->world > 0x7fffffffLL) return NN_FAIL(NN_ERR_ARG, "%s: bad n_local=%d", who, n_local);
    nnb::GatherSignal sig = {};
    sig.world = c->world;
    sig.rank = c->rank;
    for (int g = 0; g < c->world; ++g) sig.flags[g] = (unsigned*)c->symm[0].base[g];
    sig.epoch = c->epochs + 3;  // picks sent
    sig.done = nullptr;         // no flag exchange: the key word is its own arrival mark
    // the block that finishes the projection's arg-max leaves this rank's key with every rank;
    // the pick kernel, already spinning by then, takes the best of the G keys
    int rc = nnb::linear_argmax(c->ctx, n_local, K, x, W, logits_local, out_idx, c->rank * n_local, &sig, who);
    if (rc) return rc;
    COMM_CUDA(nnb::launch_comm_pick(c->flags, c->world, c->epochs + 4, 2000, c->ctx->status_dev, c->ctx->use_pdl, (int*)out_idx, c->ctx->stream));
    c->ctx->launches++;
    return NN_OK;
}

extern "C" int nn_linear_argmax_sharded_rows(nn_comm* c, int M, int n_local, int K, nn_buf x, nn_buf W, nn_buf logits_local, nn_buf out_idx) {
    const char* who = "nn_linear_argmax_sharded_rows";
    if (!c || !out_idx || !logits_local) return NN_FAIL(NN_ERR_ARG, "%s: null argument (the local logits are needed: the pick reads them)", who);
    if (!c->flags) return NN_FAIL(NN_ERR_ARG, "%s: no symmetric buffer has been allocated on this communicator", who);
    if (M < 1 || M > nnb::ROW_KEYS_MAX) return NN_FAIL(NN_ERR_ARG, "%s: M=%d outside 1..%d", who, M, nnb::ROW_KEYS_MAX);
    if (n_local <= 0 || (long long)n_local * c->world > 0x7fffffffLL) return NN_FAIL(NN_ERR_ARG, "%s: bad n_local=%d", who, n_local);
    if (c->row_keys < 0) {   // first use: the key tables (collective, like every symmetric allocation)
        if (c->ctx->capturing) return NN_FAIL(NN_ERR_UNSUPPORTED, "%s: make the first call outside a recording (it allocates the key tables)", who);
        SymmAlloc kt;
        int rc = symm_alloc(c, nnb::ROW_KEYS_BYTES, &kt);
        if (rc) return rc;
        c->symm.push_back(kt);
        c->row_keys = (int)c->symm.size() - 1;
    }
    // the projection of this rank's rows, into ordinary local memory
    int rc = nnb::linear_to_peers(c->ctx, M, n_local, K, x, W, logits_local, nullptr, 0, nullptr, who);
    if (rc) return rc;
    nnb::RowKeyTables kt = {};
    kt.world = c->world;
    kt.rank = c->rank;
    for (int g = 0; g < c->world; ++g) kt.table[g] = (unsigned long long*)c->symm[c->row_keys].base[g];
    COMM_CUDA(nnb::launch_rows_keys((const uint16_t*)logits_local, M, n_local, c->rank * n_local, kt, c->epochs + 5, c->ctx->stream));
    COMM_CUDA(nnb::launch_rows_pick(kt.table[c->rank], c->world, M, c->epochs + 5, 2000, c->ctx->status_dev, (int*)out_idx, c->ctx->stream));
    c->ctx->launches += 2;
    return NN_OK;
}

extern "C" int nn_comm_pick_unsent(nn_comm* c, unsigned timeout_ms, nn_buf out_idx) {
    if (!c || !out_idx) return NN_FAIL(NN_ERR_ARG, "nn_comm_pick_unsent: null argument");
    if (!c->flags) return NN_FAIL(NN_ERR_ARG, "nn_comm_pick_unsent: no symmetric buffer has been allocated on this communicator");
    if (timeout_ms == 0 || timeout_ms > 10000) return NN_FAIL(NN_ERR_ARG, "nn_comm_pick_unsent: timeout %u ms outside 1..10000", timeout_ms);
    // one pick round counted on both sides (sent and waited) in which no key is stored anywhere
    COMM_CUDA(nnb::launch_comm_count(c->epochs + 3, c->ctx->stream));
    COMM_CUDA(nnb::launch_comm_pick(c->flags, c->world, c->epochs + 4, timeout_ms, c->ctx->status_dev, false, (int*)out_idx, c->ctx->stream));
    c->ctx->launches += 2;
    return NN_OK;
}

extern "C" int nn_comm_all_gather(nn_comm* c, nn_buf send, nn_buf recv, size_t bytes) {
    if (!c || !send || !recv) return NN_FAIL(NN_ERR_ARG, "nn_comm_all_gather: null argument");
    if (c->world == 1) {
        if (send != recv && bytes) {
            cudaError_t e = cudaMemcpyAsync(recv, send, bytes, cudaMemcpyDeviceToDevice, c->ctx->stream);
            if (e != cudaSuccess) return NN_FAIL(NN_ERR_CUDA, "nn_comm_all_gather: %s", cudaGetErrorString(e));
        }
        return NN_OK;
    }
    const int rc = g_nccl.all_gather(send, recv, bytes, /*ncclInt8*/ 0, c->comm, c->ctx->stream);
    if (rc != 0) return NN_FAIL(NN_ERR_COMM, "ncclAllGather: %s", nccl_err(rc));
    return NN_OK;
}

extern "C" int nn_comm_free(nn_comm* c) {
    if (!c) return NN_OK;
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    for (SymmAlloc& sa : c->symm) symm_close_peers(c, sa);
    ranks_barrier(c);
    for (SymmAlloc& sa : c->symm) symm_free_local(c, sa);
    if (c->epochs) cudaFree(c->epochs);
    if (c->comm && g_nccl.comm_destroy) g_nccl.comm_destroy(c->comm);
    delete c;
    return NN_OK;
}
