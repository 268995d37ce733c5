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

#include "../../include/nnopt_b200.h"
#include "internal.h"

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
    const char* names[4] = {getenv("NNB_NCCL_LIB"), "libnccl.so.2", "libnccl.so", nullptr};
    void* h = nullptr;
    for (int i = 0; i < 3 && !h; ++i)
        if (names[i] && names[i][0]) h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
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

struct nn_comm {
    nn_context* ctx = nullptr;
    void* comm = nullptr;
    int rank = 0, world = 1;
};

extern "C" int nn_comm_unique_id(void* out) {
    if (!out) return NN_FAIL(NN_ERR_ARG, "nn_comm_unique_id: null argument");
    if (!load_nccl()) return NN_FAIL(NN_ERR_COMM, "NCCL could not be loaded (set NNB_NCCL_LIB to libnccl.so.2): %s", dlerror());
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
        if (!load_nccl()) { delete c; return NN_FAIL(NN_ERR_COMM, "NCCL could not be loaded (set NNB_NCCL_LIB to libnccl.so.2)"); }
        NcclId id;
        memcpy(id.bytes, id_bytes, sizeof(id.bytes));
        cudaSetDevice(ctx->device);
        const int rc = g_nccl.comm_init_rank(&c->comm, world, id, rank);
        if (rc != 0) { delete c; return NN_FAIL(NN_ERR_COMM, "ncclCommInitRank: %s", nccl_err(rc)); }
    }
    *out = c;
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
    if (c->comm && g_nccl.comm_destroy) g_nccl.comm_destroy(c->comm);
    delete c;
    return NN_OK;
}
